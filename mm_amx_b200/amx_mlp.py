"""The reference's torch extension surface (`amx_mlp`, torch-ext/amx_mlp.cpp:795-804) on the GPU library.

    LinearNxN()                     .set_weight(W[N,K] bf16)  .forward(x[M,K] bf16, y[M,N] fp32)  .name  deepcopy
    clflush(tensor)                 flushes the cache that holds the tensor (here: L2) so the next op starts cold
    MLP(gate, up, down)             fused Llama MLP (AMX_MLP::MLP of tests/amx-mlp.cpp), forward(x) -> bf16

Tensors may live on the CPU (the reference's case: operands are staged through the `_host` entry points and the
result is in `y` when forward returns) or on the CUDA device (no copies, asynchronous on the current stream).
Violated preconditions raise RuntimeError, like the reference's ASSERT (torch-ext/amx_mlp.cpp:23-25).
There is no CPU computation in this module.
"""
import torch

from . import capi


def _require(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream if t.is_cuda else None


class LinearNxN:
    def __init__(self):
        self.name = ""
        self._w = None
        self._cuda = False
        self.N = self.K = 0

    def set_weight(self, weight):
        """weight: [N, K] bf16, 2-D, N % 32 == 0 and K % 32 == 0 (torch-ext/amx_mlp.cpp:469-485)."""
        _require(weight.dtype == torch.bfloat16, "weight must be bfloat16")
        _require(weight.dim() == 2, "weight must be 2-D")
        N, K = weight.shape
        _require(N % 32 == 0 and K % 32 == 0, "N and K must be multiples of 32")
        _require(weight.stride(1) == 1, "weight rows must be contiguous")
        self._w = capi.Weight(weight.data_ptr(), capi.BF16, K, N, weight.stride(0) * 2, True, capi.PACK_PLAIN, None,
                              _stream(weight))
        self._cuda = weight.is_cuda
        self.N, self.K = N, K

    def forward(self, x, y):
        """y[M, N] (fp32, preallocated) = x[M, K] (bf16) @ W^T (torch-ext/amx_mlp.cpp:452-462)."""
        _require(self._w is not None, "set_weight first")
        _require(x.dim() == 2 and x.shape[1] == self.K, "x must be [M, %d]" % self.K)
        _require(x.dtype == torch.bfloat16 and y.dtype == torch.float32, "x must be bfloat16 and y float32")
        _require(tuple(y.shape) == (x.shape[0], self.N), "y must be [M, %d]" % self.N)
        _require(x.stride(1) == 1 and y.stride(1) == 1, "rows must be contiguous")
        _require(x.is_cuda == y.is_cuda, "x and y must live in the same kind of memory")
        ep = capi.make_epilogue(y.data_ptr(), y.stride(0) * 4, capi.F32)
        if x.is_cuda:
            self._w.matmul(x.data_ptr(), capi.BF16, x.shape[0], self.K, x.stride(0) * 2, ep, stream=_stream(x))
        else:
            self._w.matmul_host(x.data_ptr(), capi.BF16, x.shape[0], self.K, x.stride(0) * 2, ep)

    def __deepcopy__(self, memo):
        """Clones the PACKED weights, like the reference (torch-ext/amx_mlp.cpp:499-510); nothing is re-packed and the
        original tensor is not kept alive for it."""
        other = LinearNxN()
        other.name = self.name
        if self._w is not None:
            other._w = capi.Weight.from_blob(self._w.export())
            other._cuda, other.N, other.K = self._cuda, self.N, self.K
        return other

    def packed_state(self):
        """The packed weights as a uint8 tensor (for torch.save); load_packed_state() restores them without packing."""
        _require(self._w is not None, "set_weight first")
        return torch.frombuffer(self._w.export(), dtype=torch.uint8).clone()

    def load_packed_state(self, state):
        _require(state.dtype == torch.uint8 and state.dim() == 1, "state must be the 1-D uint8 tensor of packed_state()")
        w = capi.Weight.from_blob(state.cpu().contiguous().numpy().tobytes())
        info = w.info()
        _require(info["dtype"] == capi.BF16 and not info["compressed"], "state does not hold bf16 weights")
        self._w, self.N, self.K = w, info["N"], info["K"]


def clflush(x):
    """Makes the next access to x (and everything else) miss the GPU's L2, the role of the reference's clflush loop
    (torch-ext/amx_mlp.cpp:514-522)."""
    _require(x.is_contiguous(), "tensor must be contiguous")
    capi.flush_l2(_stream(x))


class MLP:
    """Fused Llama MLP: forward(x) = down(silu(x @ gate^T) * (x @ up^T)); weights in torch nn.Linear layout."""

    def __init__(self, gate, up, down):
        for t in (gate, up, down):
            _require(t.dtype == torch.bfloat16 and t.dim() == 2 and t.is_contiguous(), "weights must be contiguous bf16 2-D")
        N, K = gate.shape
        _require(tuple(up.shape) == (N, K) and tuple(down.shape) == (K, N), "need gate/up [N,K] and down [K,N]")
        self.K, self.N = K, N
        self._mlp = capi.Mlp(gate.data_ptr(), up.data_ptr(), down.data_ptr(), K, N, 0, 1, _stream(gate))

    def forward(self, x, out=None):
        _require(x.dim() == 2 and x.shape[1] == self.K and x.dtype == torch.bfloat16 and x.stride(1) == 1,
                 "x must be [M, %d] bf16 with contiguous rows" % self.K)
        M = x.shape[0]
        if out is None:
            out = torch.empty((M, self.K), dtype=torch.bfloat16, device=x.device)
        _require(tuple(out.shape) == (M, self.K) and out.dtype == torch.bfloat16 and out.is_cuda == x.is_cuda,
                 "out must be [M, %d] bf16 beside x" % self.K)
        if x.is_cuda:
            self._mlp.run(x.data_ptr(), x.stride(0) * 2, M, out.data_ptr(), out.stride(0) * 2, _stream(x))
        else:
            self._mlp.run_host(x.data_ptr(), x.stride(0) * 2, M, out.data_ptr(), out.stride(0) * 2)
        return out

    __call__ = forward
