// Measures what one tcgen05.mma instruction (cta_group::1, kind::f16, M = 128, K = 16) costs on the tensor
// pipe, by N and by where the A operand lives.  The prefill kernels are designed around this number: on
// B200 it is at least ~96 clocks whatever N is, so a kernel's MMA instruction count per key bounds it.
// (No counterpart in the reference: its kernels leave instruction selection to TileLang.)
#include "tb200_tcgen05.cuh"

namespace tb200 {
namespace {

constexpr int kProbeSmem = 100 * 1024;

__global__ void __launch_bounds__(128, 1) mma_issue_probe_kernel(long long* out, int n, int ts_form, int reps) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  __shared__ uint64_t bar_mem;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort, s_status;
  const uint32_t bar = smem_u32(&bar_mem);
  // operands: every element 1.0 (f16); A = 128 rows x 128 elements, B = up to 256 rows x 128 elements
  for (int i = threadIdx.x; i < 96 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) { mbar_init(bar, 1); s_abort = 0; s_status = 0; mbar_fence_init(); }
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(512u));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  if (threadIdx.x == 0) {
    const uint64_t da = make_desc(sbase, 16, 1024);
    const uint64_t db = make_desc(sbase + 32768, 16, 1024);
    const uint64_t b_panel = uint64_t(n) * 128 >> 4;          // the second 64-element panel of B
    const uint32_t idesc = make_idesc(0, 0, n);
    const long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t b = db + (kk >> 2) * b_panel + (kk & 3) * 2;
        if (ts_form) tc_mma_ts(tmem, tmem + 448 + (kk & 3) * 8, b, idesc, (r | kk) ? 1u : 0u);
        else tc_mma_ss(tmem, da + (((kk >> 2) * 16384 + (kk & 3) * 32) >> 4), b, idesc, (r | kk) ? 1u : 0u);
      }
    }
    const long long t1 = clock64();
    tc_commit(bar);
    const bool ok = mbar_wait_bounded(bar, 0, &s_abort, &s_status, 901, 2000000000LL);
    const long long t2 = clock64();
    if (blockIdx.x == 0) {
      out[0] = t1 - t0;              // clocks until the last MMA was accepted
      out[1] = ok ? t2 - t0 : -1;    // clocks until the last MMA completed (-1: the bounded wait ran out)
    }
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u));
  }
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" int tb200_mma_issue_probe(int64_t* out_clocks, int n, int a_in_tmem, int repetitions, void* stream) {
  if (!out_clocks) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "out_clocks must be a device pointer to two int64");
  if (n != 64 && n != 128 && n != 256) TB200_FAIL(TB200_ERR_UNSUPPORTED, "n must be 64, 128 or 256");
  if (repetitions <= 0 || repetitions > 100000) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "repetitions must be in [1, 100000]");
  static thread_local bool configured[64] = {false};
  int dev = 0;
  TB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) TB200_FAIL(TB200_ERR_UNSUPPORTED, "device index %d is outside [0, 64)", dev);
  if (!configured[dev]) {
    TB200_CUDA_CHECK(cudaFuncSetAttribute(mma_issue_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kProbeSmem));
    configured[dev] = true;
  }
  mma_issue_probe_kernel<<<sm_count(), 128, kProbeSmem, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<long long*>(out_clocks), n, a_in_tmem ? 1 : 0, repetitions);
  TB200_CUDA_CHECK(cudaGetLastError());
  return TB200_OK;
}
