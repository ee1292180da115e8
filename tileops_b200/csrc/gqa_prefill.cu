// placeholder until the tcgen05 prefill kernel lands
#include "tb200_common.cuh"
using namespace tb200;
extern "C" size_t tb200_gqa_prefill_workspace_bytes(int, int, int, int, int, int) { return 0; }
extern "C" int tb200_gqa_prefill(const void*, const void*, const void*, void*, float*, int, int, int, int, int,
                                 int, int, int, float, float, void*, size_t, void*) {
  TB200_FAIL(TB200_ERR_UNSUPPORTED, "prefill kernel not built yet");
}
