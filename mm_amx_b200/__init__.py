"""B200 (sm_100a) implementation of the fully-connected / Llama-MLP hot path of usstq/mm_amx.

    mm_amx_b200.capi      ctypes binding of the C ABI declared in include/b200fc.h
    mm_amx_b200.amx_mlp   the reference's torch extension surface (LinearNxN, clflush) plus the fused MLP
    mm_amx_b200.tp        Megatron-style tensor-parallel MLP over torch.distributed
    mm_amx_b200.build     builds libb200fc.so in-tree with nvcc

The compute path is the CUDA library only; importing the binding fails loudly when it has not been built.
"""
