"""memfabric-b200: a Blackwell-native memory-fabric library.

Python surface of the reference's ``memfabric_hybrid`` package
(src/smem/python/memfabric_hybrid/memfabric_hybrid/__init__.py:36-68): module-level
``initialize / uninitialize / set_log_level / set_extern_logger / get_last_err_msg /
get_and_clear_last_err_msg / set_conf_store_tls / set_conf_store_tls_key / create_config_store``,
the ``bm`` and ``shm`` submodules and ``TransferEngine``. On top of that: ``native`` (control-plane
classes and raw kernel launchers), ``ops`` (torch-facing fused kernels), ``parallel`` (process-group
helpers over the symmetric heap), ``models`` (workload shapes) and ``utils``.
"""
from ._loader import _pymf

initialize = _pymf.initialize
uninitialize = _pymf.uninitialize
set_log_level = _pymf.set_log_level
set_extern_logger = _pymf.set_extern_logger
get_last_err_msg = _pymf.get_last_err_msg
get_and_clear_last_err_msg = _pymf.get_and_clear_last_err_msg
set_conf_store_tls = _pymf.set_conf_store_tls
set_conf_store_tls_key = _pymf.set_conf_store_tls_key
create_config_store = _pymf.create_config_store
destroy_config_store = _pymf.destroy_config_store
version = _pymf.version
trace_enable = _pymf.trace_enable
trace_disable = _pymf.trace_disable
trace_dump = _pymf.trace_dump

bm = _pymf.bm
native = _pymf.native
shm = getattr(_pymf, "shm", None)
TransferEngine = getattr(_pymf, "TransferEngine", None)
TransferOpcode = getattr(_pymf, "TransferOpcode", None)
TransDataOpType = getattr(_pymf, "TransDataOpType", None)



def get_include_path() -> str:
    """Directory of the public C / CUDA headers (`mf/*.h`, `mf/device/*.cuh`): the package's own copy when installed from a
    release, the repository's `include/` when run from a source tree."""
    import os

    here = os.path.dirname(os.path.abspath(__file__))
    packaged = os.path.join(here, "include")
    return packaged if os.path.isdir(packaged) else os.path.join(os.path.dirname(here), "include")


def get_lib_path() -> str:
    """Directory that holds libmf_core.so."""
    import os

    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib")


__all__ = [
    "get_include_path", "get_lib_path",
    "initialize", "uninitialize", "set_log_level", "set_extern_logger", "get_last_err_msg",
    "get_and_clear_last_err_msg", "set_conf_store_tls", "set_conf_store_tls_key", "create_config_store",
    "destroy_config_store", "version", "bm", "shm", "native", "TransferEngine", "TransferOpcode",
    "TransDataOpType", "trace_enable", "trace_disable", "trace_dump",
]
