"""so3lr_b200: B200-native (sm_100a) energy + force evaluation for the SO3LR force field.

The public names mirror the reference package (so3lr/__init__.py:3-7).  Importing the package loads
libso3lr_b200.so; it fails loudly when the library has not been built.
"""
__version__ = "0.1.0"

from .engine import Model, System  # noqa: F401
from .api import make_ase_calculator as So3lrCalculator  # noqa: F401
from .api import Graph  # noqa: F401
from .api import to_jax_md  # noqa: F401
from .api import make_potential_fn as So3lrPotential  # noqa: F401
from .api import make_so3lr as So3lr  # noqa: F401
from .api import neighbor_list  # noqa: F401
