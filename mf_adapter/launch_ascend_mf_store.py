"""Stand-alone config store under the reference's module name: the URL comes from the command line, MF_STORE_URL or
ASCEND_MF_STORE_URL (see memfabric_hybrid_b200.launch_store)."""
import sys

from memfabric_hybrid_b200.launch_store import main

if __name__ == "__main__":
    sys.exit(main())
