"""so3lr_b200: B200-native (sm_100a) energy + force evaluation for the SO3LR force field.

The public names mirror the reference package (so3lr/__init__.py:3-7).  Importing the package loads
libso3lr_b200.so; it fails loudly when the library has not been built.
"""
__version__ = "0.1.0"

from .engine import Model, System  # noqa: F401
