"""symmetrix_b200: B200-native MACE energy+force evaluation behind the interface of wcwitt/symmetrix."""
from .mace import MACE, MACEKokkos, MACEKokkosFloat, SymmetrixError  # noqa: F401
from .calculator import Symmetrix  # noqa: F401
