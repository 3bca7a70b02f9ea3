"""Where the Forward reference tree is, if it is anywhere (test infrastructure).

FWD_REFERENCE_ROOT names it; without the variable a directory called `reference` beside this
repository is taken when it looks like a Forward checkout.  None means "not here": callers skip
whatever needs the tree (building the reference's kernels, regenerating golden files, the tests
that re-read the reference's own fixtures)."""
import os

_HERE = os.path.dirname(os.path.abspath(__file__))


def reference_root():
    root = os.environ.get("FWD_REFERENCE_ROOT")
    if not root:
        root = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    marker = os.path.join(root, "source", "trt_engine", "trt_network_crt", "plugins", "embedding_bag_plugin")
    return root if os.path.isdir(marker) else None
