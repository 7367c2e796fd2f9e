"""TEST INFRASTRUCTURE: CPU oracle for the mm_amx fully-connected hot path.

Only tests/, __graft_entry__.smoke() and the CPU-baseline legs of bench.py may import this package.

    oracle.port  plain C++ restatement (oracle/oracle.cpp), runs on any host
    oracle.ref   the reference's own AMX kernels behind a C shim (oracle/ref_harness.cpp), AMX hosts only
"""
