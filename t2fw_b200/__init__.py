"""t2fw_b200: the fast-weight recurrences of T2FW (decay rule "LFW", delta rule "DFW") as
hand-written sm_100a CUDA behind the reference's Python API.

    from t2fw_b200.functional_lfw import LFWFunction
    from t2fw_b200.functional_dfw import DFWFunction

The native libraries are built ahead of time (python -m t2fw_b200.build) and loaded on first
use; there is no CPU or PyTorch fallback: if the libraries are missing the import fails.
"""
__version__ = "0.1.0"
