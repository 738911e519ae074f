"""Drop-in name for programs written against the reference's Python package: `import memfabric_hybrid` gives the same names
(`bm`, `shm`, `TransferEngine`, `TransferOpcode`, `initialize`, `set_log_level`, ..., `get_include_path`, `get_lib_path`;
src/smem/python/memfabric_hybrid/memfabric_hybrid/__init__.py:36-68 of the reference), served by memfabric_hybrid_b200."""
from memfabric_hybrid_b200 import *  # noqa: F401,F403
from memfabric_hybrid_b200 import __all__  # noqa: F401
