"""Drop-in name for the reference's transfer-engine-only package (src/smem/python/mk_transfer_adapter/mf_adapter/__init__.py:
`TransferEngine`, `set_log_level`, `create_config_store`, `set_conf_store_tls`), served by memfabric_hybrid_b200.
`python -m mf_adapter.launch_ascend_mf_store` starts a stand-alone store like the reference's launcher of that name."""
from memfabric_hybrid_b200 import TransferEngine, create_config_store, set_conf_store_tls, set_log_level  # noqa: F401

__all__ = ["TransferEngine", "set_log_level", "create_config_store", "set_conf_store_tls"]
