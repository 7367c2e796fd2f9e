"""Megatron-style tensor-parallel Llama MLP: one process per GPU, one all-reduce on the down-projection output.

Three ways to do that all-reduce: PullFusedTensorParallelMLP (inside the down-projection kernel; the fastest, needs
torch symmetric memory with an NVLink multicast mapping), TensorParallelMLP (torch.distributed: NCCL on GPUs, gloo in
the CPU tests), FusedTensorParallelMLP (multimem.red from the epilogue).

The reference shards the same way across CPU cores: gate/up by output channels (Linear::setup, tests/amx-mlp.cpp:554-593)
and the down projection by K with an fp32 add of the partial results before the bf16 rounding (:559-589, :656-683).
Here rank r keeps rows [r*N/t, (r+1)*N/t) of gate and up and the same columns of down; every rank computes its
contribution to out[M, K]; one torch.distributed all-reduce (NCCL over NVLink on GPUs) sums them.

  partial dtype "f32": contributions are summed in fp32 and rounded to bf16 once, like the reference's split-K.
  partial dtype "bf16": contributions are rounded to bf16 first (half the bytes on the wire); the sum of t bf16
                        values stays within the 1e-2 bound of the bf16 paths.

The local computation is the CUDA library (capi.Mlp).  `local` can be replaced by another object with the same
run_partial() signature; the CPU tests use that to check the sharding and reduction logic under gloo.
"""
import torch
import torch.distributed as dist

from . import capi


def shard_rows(n_total, rank, world):
    """Row range of gate/up (= column range of down) owned by `rank`; N must divide evenly, in 32-row units."""
    if n_total % world:
        raise ValueError("intermediate size %d is not divisible by tensor-parallel size %d" % (n_total, world))
    ns = n_total // world
    if ns % 32:
        raise ValueError("per-rank intermediate size %d must be a multiple of 32" % ns)
    return rank * ns, (rank + 1) * ns


class CudaLocalMLP:
    """This rank's shard on its GPU.  gate/up: [N, K], down: [K, N] bf16 torch tensors (CPU or CUDA), FULL matrices."""

    def __init__(self, gate, up, down, rank, world):
        N, K = gate.shape
        assert up.shape == (N, K) and down.shape == (K, N)
        for t in (gate, up, down):
            assert t.dtype == torch.bfloat16 and t.is_contiguous()
        shard_rows(N, rank, world)
        self.K, self.N, self.world = K, N, world
        self.mlp = capi.Mlp(gate.data_ptr(), up.data_ptr(), down.data_ptr(), K, N, rank, world,
                            torch.cuda.current_stream().cuda_stream)

    def run_partial(self, x, out):
        """x [M, K] bf16 CUDA; out [M, K] fp32 or bf16 CUDA: this rank's contribution."""
        dt = capi.F32 if out.dtype == torch.float32 else capi.BF16
        self.mlp.run_partial(x.data_ptr(), x.stride(0) * 2, x.shape[0], out.data_ptr(), dt,
                             out.stride(0) * out.element_size(), torch.cuda.current_stream().cuda_stream)

    def gate_up(self, x):
        self.mlp.gate_up(x.data_ptr(), x.stride(0) * 2, x.shape[0], torch.cuda.current_stream().cuda_stream)

    def down_rows(self, row0, rows, out):
        """out [rows, K]: this rank's contribution for rows [row0, row0 + rows) of the last gate_up."""
        dt = capi.F32 if out.dtype == torch.float32 else capi.BF16
        self.mlp.down_rows(row0, rows, out.data_ptr(), dt, out.stride(0) * out.element_size(),
                           torch.cuda.current_stream().cuda_stream)


class TensorParallelMLP:
    def __init__(self, local, K, group=None, partial_dtype=torch.float32, chunk_rows=0):
        """local: object with run_partial(x, out); chunk_rows > 0 splits M so that the all-reduce of one chunk overlaps
        the computation of the next (CUDA only)."""
        self.local, self.K, self.group = local, K, group
        self.partial_dtype = partial_dtype
        self.chunk_rows = chunk_rows
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self._comm_stream = None

    def _round(self, partial, out):
        if partial.dtype == torch.bfloat16:
            if out.data_ptr() != partial.data_ptr():
                out.copy_(partial)
        elif partial.is_cuda:
            capi.add_round_bf16(partial.data_ptr(), None, out.data_ptr(), partial.numel(),
                                torch.cuda.current_stream().cuda_stream)
        else:
            out.copy_(partial.to(torch.bfloat16))  # round to nearest even, CPU test path only

    def forward(self, x, out=None, partial=None):
        """x [M, K] bf16 (replicated on every rank) -> out [M, K] bf16 (identical on every rank)."""
        M = x.shape[0]
        if out is None:
            out = torch.empty((M, self.K), dtype=torch.bfloat16, device=x.device)
        if partial is None:
            partial = out if self.partial_dtype == torch.bfloat16 else torch.empty((M, self.K), dtype=torch.float32,
                                                                                   device=x.device)
        chunk = self.chunk_rows if (self.chunk_rows and self.world > 1) else M
        if chunk >= M:
            self.local.run_partial(x, partial)
            if self.world > 1:
                dist.all_reduce(partial, group=self.group)
            self._round(partial, out)
            return out
        # chunked: the collective of finished rows runs on a side stream while the following rows are multiplied
        # (CUDA; on CPU tensors the same row blocks are reduced one after the other).
        # When the local object can run the two stages separately, gate/up runs once over all rows (full GEMM waves)
        # and only the down projection is cut into row blocks; otherwise whole forwards are chunked.
        overlap = x.is_cuda
        if overlap:
            if self._comm_stream is None:
                self._comm_stream = torch.cuda.Stream()
            cur = torch.cuda.current_stream()
        staged = hasattr(self.local, "gate_up") and hasattr(self.local, "down_rows")
        if staged:
            self.local.gate_up(x)
        for m0 in range(0, M, chunk):
            m1 = min(M, m0 + chunk)
            if staged:
                self.local.down_rows(m0, m1 - m0, partial[m0:m1])
            else:
                self.local.run_partial(x[m0:m1], partial[m0:m1])
            if overlap:
                ev = torch.cuda.Event()
                ev.record(cur)
                with torch.cuda.stream(self._comm_stream):
                    self._comm_stream.wait_event(ev)
                    dist.all_reduce(partial[m0:m1], group=self.group)
            else:
                dist.all_reduce(partial[m0:m1], group=self.group)
        if overlap:
            cur.wait_stream(self._comm_stream)
        self._round(partial, out)
        return out


class FusedTensorParallelMLP:
    """Tensor-parallel MLP whose all-reduce happens inside the down-projection kernel.

    The output lives in a torch symmetric-memory buffer that every rank maps through one NVLink multicast (NVLS)
    address.  The GEMM epilogue adds each rank's contribution into all replicas with `multimem.red`
    (b200fc_mlp_down_reduce), so the transfer overlaps the math tile by tile and no collective kernel runs.
    Per step and rank:  zero own replica -> barrier -> gate/up -> down + in-switch reduce -> barrier.
    Every replica receives every rank's contribution (ingress = world x output bytes) and the in-switch atomics slow
    the epilogue; PullFusedTensorParallelMLP below moves the optimal number of bytes and measured faster at every
    group size.
    Needs M > 16 and a CUDA build of torch with symmetric memory + multicast support.
    """

    def __init__(self, mlp, K, max_M, group=None, out_dtype=torch.bfloat16):
        """mlp: capi.Mlp holding this rank's shard (created with tp_rank / tp_size, or from pre-sharded weights)."""
        import torch.distributed._symmetric_memory as symm_mem
        self.mlp, self.K, self.max_M = mlp, K, max_M
        self.group = group if group is not None else dist.group.WORLD
        self.out_dtype = out_dtype
        dev = torch.device("cuda", torch.cuda.current_device())
        self.buf = symm_mem.empty((max_M, K), dtype=out_dtype, device=dev)
        self.handle = symm_mem.rendezvous(self.buf, self.group.group_name)
        if not self.handle.multicast_ptr:
            raise RuntimeError("this system offers no NVLink multicast mapping for symmetric memory")

    def forward(self, x):
        """x [M, K] bf16 CUDA (replicated) -> view of the symmetric buffer [M, K] holding the reduced result.
        The view is overwritten by the next forward."""
        M = x.shape[0]
        if not (16 < M <= self.max_M):
            raise ValueError("M must be in (16, %d]" % self.max_M)
        stream = torch.cuda.current_stream().cuda_stream
        out = self.buf[:M]
        out.zero_()
        self.handle.barrier(channel=0)          # every replica is zero before anybody adds into it
        self.mlp.gate_up(x.data_ptr(), x.stride(0) * 2, M, stream)
        dt = capi.F32 if self.out_dtype == torch.float32 else capi.BF16
        self.mlp.down_reduce(M, self.handle.multicast_ptr, dt, self.K * self.buf.element_size(), stream)
        self.handle.barrier(channel=1)          # all contributions have landed in every replica
        return out


class PullFusedTensorParallelMLP:
    """Tensor-parallel MLP whose all-reduce is done by the down-projection kernel itself, pull style
    (b200fc_mlp_down_allreduce): multiplying CTA pairs store bf16 tiles into a symmetric partial buffer and signal the
    tile's owner; a few SMs of the same grid pull finished tiles from all ranks with multimem.ld_reduce (summed in the
    NVSwitch) and multicast the sums into every rank's output with multimem.st.  One symmetric-memory barrier per step.
    """

    MAX_TILES = 8192

    def __init__(self, mlp, K, max_M, group=None, comm_sms=8):
        import torch.distributed._symmetric_memory as symm_mem
        self.mlp, self.K, self.max_M, self.comm_sms = mlp, K, max_M, comm_sms
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        dev = torch.device("cuda", torch.cuda.current_device())
        name = self.group.group_name
        self.partial = symm_mem.empty((max_M, K), dtype=torch.bfloat16, device=dev)
        self.out = symm_mem.empty((max_M, K), dtype=torch.bfloat16, device=dev)
        self.flags = symm_mem.empty((2, self.MAX_TILES), dtype=torch.int32, device=dev)  # two arrays, used alternately
        self.h_partial = symm_mem.rendezvous(self.partial, name)
        self.h_out = symm_mem.rendezvous(self.out, name)
        self.h_flags = symm_mem.rendezvous(self.flags, name)
        if not (self.h_partial.multicast_ptr and self.h_out.multicast_ptr):
            raise RuntimeError("this system offers no NVLink multicast mapping for symmetric memory")
        self.flags.zero_()
        torch.cuda.synchronize()
        self.h_flags.barrier(channel=0)
        self.parity = 0

    def forward(self, x):
        """x [M, K] bf16 CUDA (replicated) -> view [M, K] of the symmetric output buffer (valid until the next call)."""
        M = x.shape[0]
        if not (16 < M <= self.max_M):
            raise ValueError("M must be in (16, %d]" % self.max_M)
        stream = torch.cuda.current_stream().cuda_stream
        p = self.parity
        # Clear the counters of the NEXT step now: nobody signals them before the barrier that ends this step, and this
        # rank passes that barrier only after this memset.
        self.flags[1 - p].zero_()
        self.mlp.gate_up(x.data_ptr(), x.stride(0) * 2, M, stream)
        ar = capi.AllReduce()
        ar.world, ar.rank = self.world, self.rank
        ar.partial_local = self.partial.data_ptr()
        ar.partial_mc = self.h_partial.multicast_ptr
        ar.out_mc = self.h_out.multicast_ptr
        ar.ld_bytes = self.K * 2
        for r in range(self.world):
            ar.flags[r] = self.h_flags.buffer_ptrs[r] + p * self.MAX_TILES * 4
        ar.max_tiles = self.MAX_TILES
        ar.comm_sms = self.comm_sms
        self.mlp.down_allreduce(M, ar, stream)
        self.h_out.barrier(channel=1)   # every rank's tiles have been reduced and multicast
        self.parity = 1 - p
        return self.out[:M]
