"""santa_b200 -- B200 (sm_100a) S2ANTA decode attention behind the reference's operator surface.

``santa_b200.ops`` is the Python host mirror over the C ABI; the drop-in extension
modules ``santa_flash_batch_cuda`` / ``santa_prop_batch_cuda`` live in ``santa_b200/lib``
(``santa_b200.enable_dropin()`` puts that directory on ``sys.path``).
"""
import os
import sys

__all__ = ["enable_dropin", "LIB_DIR"]

LIB_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib")


def enable_dropin() -> str:
    """Make ``import santa_flash_batch_cuda`` / ``import santa_prop_batch_cuda`` resolve to this build."""
    if LIB_DIR not in sys.path:
        sys.path.insert(0, LIB_DIR)
    return LIB_DIR
