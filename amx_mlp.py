"""`import amx_mlp` — the module name of the reference's torch extension (torch-ext/setup.py:10-13), so that a script
written against it (torch-ext/test.py) runs unchanged on the GPU library.  Everything lives in mm_amx_b200.amx_mlp;
this file only re-exports the bound surface of torch-ext/amx_mlp.cpp:795-804 plus the fused MLP."""
from mm_amx_b200.amx_mlp import LinearNxN, MLP, clflush  # noqa: F401

__all__ = ["LinearNxN", "MLP", "clflush"]
