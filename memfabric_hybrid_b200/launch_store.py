"""Stand-alone config store:  python -m memfabric_hybrid_b200.launch_store [tcp://ip:port]

The URL defaults to $MF_STORE_URL (the reference's launcher reads ASCEND_MF_STORE_URL,
src/smem/python/mf_adapter/launch_ascend_mf_store.py; that name is honoured too). Runs until interrupted."""
import os
import signal
import sys
import time

from . import create_config_store, destroy_config_store, set_log_level


def main() -> int:
    url = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MF_STORE_URL", os.environ.get("ASCEND_MF_STORE_URL", ""))
    if not url:
        print("usage: python -m memfabric_hybrid_b200.launch_store tcp://ip:port  (or set MF_STORE_URL)", file=sys.stderr)
        return 2
    set_log_level(int(os.environ.get("MF_LOG_LEVEL", os.environ.get("ASCEND_MF_LOG_LEVEL", "1"))))
    rc = create_config_store(url)
    if rc != 0:
        print(f"cannot start the store on {url} (rc={rc})", file=sys.stderr)
        return 1
    print(f"memfabric config store serving {url}", flush=True)
    stop = []
    signal.signal(signal.SIGTERM, lambda *_: stop.append(1))
    signal.signal(signal.SIGINT, lambda *_: stop.append(1))
    while not stop:
        time.sleep(0.2)
    destroy_config_store(url)
    return 0


if __name__ == "__main__":
    sys.exit(main())
