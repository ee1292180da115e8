from . import formulas
from .profile import available_profiles, load_profile

__all__ = ["formulas", "available_profiles", "load_profile"]
