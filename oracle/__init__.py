"""CPU oracle of the verify path: TEST INFRASTRUCTURE ONLY.

Only the tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` import this package; the
shipped library never does.  ``oracle.lib()`` is the C restatement (fnx_oracle.c), ``oracle.ref()`` the
reference's own host code behind ref_shim.cpp (None where it was not built).
"""
from .pyoracle import *  # noqa: F401,F403
