"""CPU, world_size 2 under gloo: the tensor-parallel sharding + all-reduce + rounding logic of mm_amx_b200.tp.

The local computation is replaced by the CPU oracle (test only); on GPUs it is the CUDA library.  Checks that the
summed contributions of the Megatron shards reproduce the unsharded oracle result, for fp32 and bf16 partials.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleLocal:
    """stands in for tp.CudaLocalMLP on CPU: same sharding arguments, same run_partial() contract"""

    def __init__(self, gate, up, down, rank, world):
        from mm_amx_b200 import tp
        N = gate.shape[0]
        r0, r1 = tp.shard_rows(N, rank, world)
        bits = lambda t: t.view(torch.int16).numpy().view(np.uint16)
        self.g, self.u = bits(gate)[r0:r1].copy(), bits(up)[r0:r1].copy()
        self.d = np.ascontiguousarray(bits(down)[:, r0:r1])

    def run_partial(self, x, out):
        from oracle import port
        xb = x.contiguous().view(torch.int16).numpy().view(np.uint16)
        _, part = port.mlp(xb, self.g, self.u, self.d, want_partial=True)
        self._store(part, out)

    @staticmethod
    def _store(part, out):
        from oracle import port
        if out.dtype == torch.float32:
            out.copy_(torch.from_numpy(part))
        else:
            out.copy_(torch.from_numpy(port.f32_to_bf16(part).view(np.int16)).view(torch.bfloat16))


class StagedOracleLocal(OracleLocal):
    """also offers the two stages on their own, like tp.CudaLocalMLP: gate_up() keeps the activation, down_rows()
    multiplies a block of its rows"""

    def gate_up(self, x):
        from oracle import port
        xb = x.contiguous().view(torch.int16).numpy().view(np.uint16)
        _, self.act = port.mlp(xb, self.g, self.u, self.d, want_act=True)

    def down_rows(self, row0, rows, out):
        from oracle import port
        part = port.gemm_bf16(np.ascontiguousarray(self.act[row0:row0 + rows]), np.ascontiguousarray(self.d.T))
        self._store(part, out)


def worker(rank, world, port_no, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port_no)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from mm_amx_b200 import tp
    from oracle import port
    torch.manual_seed(0)
    M, K, N = 6, 128, 256
    x = torch.randn(M, K).to(torch.bfloat16)
    gate = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    up = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    down = (torch.randn(K, N) * 0.05).to(torch.bfloat16)
    bits = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16)
    full = port.mlp(bits(x), bits(gate), bits(up), bits(down))
    full_f = (full.astype(np.uint32) << 16).view(np.float32)
    errs = []
    for pdt in (torch.float32, torch.bfloat16):
        m = tp.TensorParallelMLP(OracleLocal(gate, up, down, rank, world), K, partial_dtype=pdt)
        out = m.forward(x)
        got = (bits(out).astype(np.uint32) << 16).view(np.float32)
        errs.append(float(np.abs(got - full_f).max() / np.abs(full_f).max()))
        # every rank holds the same result
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        assert all(torch.equal(g, gathered[0]) for g in gathered)
    # row blocks: whole forwards per block, and gate/up once + the down projection per block (ragged last block)
    for local_cls in (OracleLocal, StagedOracleLocal):
        m = tp.TensorParallelMLP(local_cls(gate, up, down, rank, world), K, partial_dtype=torch.float32, chunk_rows=4)
        out = m.forward(x)
        got = (bits(out).astype(np.uint32) << 16).view(np.float32)
        errs.append(float(np.abs(got - full_f).max() / np.abs(full_f).max()))
    results[rank] = errs
    dist.destroy_process_group()


def test_tensor_parallel_mlp_world2_gloo():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port_no = 29500 + (os.getpid() % 2000)
    mp.spawn(worker, args=(world, port_no, results), nprocs=world, join=True)
    assert len(results) == world
    for r in range(world):
        e32, e16, e_blocks, e_staged = results[r]
        assert e32 < 4e-3      # fp32 partial sum, one bf16 rounding (a bf16 ulp is 2^-8 = 3.9e-3 of the value)
        assert e16 < 1e-2      # bf16 partials: the bound of the bf16 paths
        assert e_blocks == e32 and e_staged < 4e-3   # row blocks change nothing; the staged path sums the same shards


def test_shard_rows():
    from mm_amx_b200 import tp
    assert tp.shard_rows(28672, 3, 8) == (3 * 3584, 4 * 3584)
    assert tp.shard_rows(11008, 0, 1) == (0, 11008)
    with pytest.raises(ValueError):
        tp.shard_rows(11008, 0, 3)
    assert tp.shard_rows(11008, 7, 8) == (7 * 1376, 11008)   # 1376 = 43 * 32 rows per rank
    with pytest.raises(ValueError):
        tp.shard_rows(11008, 0, 16)  # 688 rows per rank, not a multiple of 32
