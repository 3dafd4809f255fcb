"""cyb_b200 — B200 (sm_100a) engine for cyb's local-LLM hot path.

The product is the CUDA library ``libqeng.so`` behind the C ABI declared in
``include/qeng.h``; ``cyb_b200.qeng`` is its ctypes binding and
``cyb_b200.soma`` the host-side mirror of the caller's interface.  Importing
``cyb_b200.qeng`` loads the library and fails loudly if it has not been built.
"""
__all__ = ["build", "qeng"]
