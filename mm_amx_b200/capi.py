"""ctypes binding of libb200fc.so (C ABI: include/b200fc.h).  No computation happens in Python."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200fc.so")

OK, ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_NOMEM, ERR_KERNEL = range(6)
BF16, S8, U8, F32, S32, S4 = range(6)
STEP_NONE, STEP_DEQUANT, STEP_BIAS, STEP_GELU, STEP_QUANT, STEP_SILU_MUL = 0, 1, 2, 4, 8, 16
PACK_PLAIN, PACK_QUANT_TENSOR, PACK_INT8_CHANNEL, PACK_INT4_GROUP = 0, 1, 2, 3
INT4_GROUP = 128

c_int, c_i64, c_float, c_void_p = ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p


class Epilogue(ctypes.Structure):
    """b200fc_epilogue_t"""
    _fields_ = [("steps", c_int), ("out_dtype", c_int), ("C", c_void_p), ("ldc_bytes", c_i64), ("bias", c_void_p),
                ("deq_scale", c_float), ("deq_scale_per_oc", c_void_p), ("q_scale", c_float),
                ("q_scale_per_oc", c_void_p)]


class AllReduce(ctypes.Structure):
    """b200fc_allreduce_t"""
    _fields_ = [("world", c_int), ("rank", c_int), ("partial_local", c_void_p), ("partial_mc", c_void_p),
                ("out_mc", c_void_p), ("ld_bytes", c_i64), ("flags", c_void_p * 8), ("max_tiles", c_int),
                ("comm_sms", c_int)]


class Attention(ctypes.Structure):
    """b200fc_attention_t"""
    _fields_ = [("B", c_int), ("H", c_int), ("Hkv", c_int), ("N", c_int), ("D", c_int), ("q", c_void_p),
                ("q_batch_stride", c_i64), ("q_head_stride", c_i64), ("k", c_void_p), ("v", c_void_p),
                ("kv_batch_stride", c_i64), ("kv_head_stride", c_i64), ("kv_token_stride", c_i64), ("out", c_void_p),
                ("out_batch_stride", c_i64), ("out_head_stride", c_i64), ("out_dtype", c_int), ("seq_lens", c_void_p),
                ("scale", c_float)]


# name -> (restype, argtypes); every symbol include/b200fc.h declares
SIGNATURES = {
    "b200fc_last_error": (ctypes.c_char_p, []),
    "b200fc_version": (ctypes.c_char_p, []),
    "b200fc_launch_count": (c_i64, []),
    "b200fc_mlp_host_plan": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int),
                                            ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.POINTER(ctypes.c_int),
                                            ctypes.POINTER(ctypes.c_int)]),
    "b200fc_sync_check": (c_int, [c_void_p]),
    "b200fc_set_wait_limit_ns": (c_int, [ctypes.c_uint64]),
    "b200fc_set_sm_limit": (c_int, [c_int]),
    "b200fc_set_decode_ctas_per_sm": (c_int, [c_int]),
    "b200fc_weight_pack": (c_int, [c_void_p, c_int, c_int, c_int, c_i64, c_int, c_int, c_void_p,
                                   ctypes.POINTER(c_void_p), c_void_p]),
    "b200fc_weight_free": (c_int, [c_void_p]),
    "b200fc_weight_info": (c_int, [c_void_p, ctypes.POINTER(c_int), ctypes.POINTER(c_int), ctypes.POINTER(c_int),
                                   ctypes.POINTER(c_int), ctypes.POINTER(c_float)]),
    "b200fc_weight_unpack": (c_int, [c_void_p, c_void_p, c_i64, c_void_p]),
    "b200fc_weight_group_scales": (c_int, [c_void_p, c_void_p, c_i64, c_void_p]),
    "b200fc_weight_export_size": (c_int, [c_void_p, ctypes.POINTER(ctypes.c_size_t)]),
    "b200fc_weight_export": (c_int, [c_void_p, c_void_p, ctypes.c_size_t, c_void_p]),
    "b200fc_weight_import": (c_int, [c_void_p, ctypes.c_size_t, ctypes.POINTER(c_void_p), c_void_p]),
    "b200fc_matmul": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_i64, c_int, c_int,
                              ctypes.POINTER(Epilogue), c_void_p]),
    "b200fc_matmul_host": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_i64, c_int, c_int,
                                   ctypes.POINTER(Epilogue), c_void_p]),
    "b200fc_matvec": (c_int, [c_void_p, c_int, c_int, c_int, c_i64, c_void_p, c_void_p, c_void_p]),
    "b200fc_matvec_host": (c_int, [c_void_p, c_int, c_int, c_int, c_i64, c_void_p, c_void_p, c_void_p]),
    "b200fc_mlp_create": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                  ctypes.POINTER(c_void_p), c_void_p]),
    "b200fc_mlp_free": (c_int, [c_void_p]),
    "b200fc_mlp_reserve": (c_int, [c_void_p, c_int]),
    "b200fc_mlp_run": (c_int, [c_void_p, c_void_p, c_i64, c_int, c_void_p, c_i64, c_void_p]),
    "b200fc_mlp_run_partial": (c_int, [c_void_p, c_void_p, c_i64, c_int, c_void_p, c_int, c_i64, c_void_p]),
    "b200fc_mlp_gate_up": (c_int, [c_void_p, c_void_p, c_i64, c_int, c_void_p]),
    "b200fc_mlp_down": (c_int, [c_void_p, c_int, c_void_p, c_int, c_i64, c_void_p]),
    "b200fc_mlp_down_rows": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_i64, c_void_p]),
    "b200fc_mlp_down_reduce": (c_int, [c_void_p, c_int, c_void_p, c_int, c_i64, c_void_p]),
    "b200fc_mlp_down_allreduce": (c_int, [c_void_p, c_int, ctypes.POINTER(AllReduce), c_void_p]),
    "b200fc_mlp_run_host": (c_int, [c_void_p, c_void_p, c_i64, c_int, c_void_p, c_i64, c_void_p]),
    "b200fc_mlp_run_decode_static": (c_int, [c_void_p, c_void_p, c_i64, c_int, c_void_p, c_int, c_i64, c_void_p]),
    "b200fc_rmsnorm": (c_int, [c_void_p, c_i64, c_int, c_int, c_void_p, ctypes.c_float, c_void_p, c_i64, c_void_p]),
    "b200fc_mlp_run_block": (c_int, [c_void_p, c_void_p, c_i64, c_int, ctypes.c_float, c_void_p, c_int, c_void_p, c_i64,
                                     c_void_p]),
    "b200fc_mlp_decode_static_capacity": (c_i64, []),
    "b200fc_mlp_decode_static_footprint": (c_i64, []),
    "b200fc_mlp_act": (c_void_p, [c_void_p]),
    "b200fc_decode_attention": (c_int, [ctypes.POINTER(Attention), c_void_p]),
    "b200fc_device_malloc": (c_int, [ctypes.POINTER(c_void_p), c_i64]),
    "b200fc_device_free": (c_int, [c_void_p]),
    "b200fc_memcpy": (c_int, [c_void_p, c_void_p, c_i64, c_void_p]),
    "b200fc_add_round_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_i64, c_void_p]),
    "b200fc_flush_l2": (c_int, [c_void_p]),
}

_LIB = None


class B200FCError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("b200fc error %d: %s" % (code, msg))
        self.code = code


def lib():
    """Loads the CUDA library.  There is no fallback: a missing library is an error."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("%s not found: build it with `python -m mm_amx_b200.build` (needs nvcc)" % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _LIB = L
    return _LIB


def check(rc):
    if rc != OK:
        raise B200FCError(rc, lib().b200fc_last_error().decode())


def last_error():
    return lib().b200fc_last_error().decode()


def launch_count():
    return lib().b200fc_launch_count()


def set_sm_limit(sms):
    check(lib().b200fc_set_sm_limit(sms))


def set_decode_ctas_per_sm(n):
    """0 = default (2); 1 lets decode kernels of different streams overlap; see include/b200fc.h."""
    check(lib().b200fc_set_decode_ctas_per_sm(n))


def sync_check(stream=None):
    check(lib().b200fc_sync_check(stream))


def set_wait_limit_ns(ns):
    """Bound of every wait inside the kernels (default 2 s); see b200fc_set_wait_limit_ns in include/b200fc.h."""
    check(lib().b200fc_set_wait_limit_ns(int(ns)))


def make_epilogue(C, ldc_bytes, out_dtype, steps=0, bias=None, deq_scale=1.0, deq_scale_per_oc=None, q_scale=1.0,
                  q_scale_per_oc=None):
    """Pointers are raw addresses (ints): device addresses for matmul, host addresses for matmul_host."""
    return Epilogue(steps, out_dtype, C, ldc_bytes, bias, deq_scale, deq_scale_per_oc, q_scale, q_scale_per_oc)


class Weight:
    """Packed weights (b200fc_weight_t): the internalB cache of amx_kernel::Matmul, resident in HBM."""

    def __init__(self, B_ptr, dtype, K, N, ldb_bytes, transposeB=False, pack_mode=PACK_PLAIN, scales_ptr=None,
                 stream=None):
        h = c_void_p()
        check(lib().b200fc_weight_pack(B_ptr, dtype, K, N, ldb_bytes, int(transposeB), pack_mode, scales_ptr,
                                       ctypes.byref(h), stream))
        self.h, self.K, self.N = h, K, N

    def info(self):
        K, N, dt, comp, sc = c_int(), c_int(), c_int(), c_int(), c_float()
        check(lib().b200fc_weight_info(self.h, K, N, dt, comp, sc))
        return {"K": K.value, "N": N.value, "dtype": dt.value, "compressed": bool(comp.value), "deq_scale": sc.value}

    def unpack(self, dst_ptr, ld_bytes, stream=None):
        check(lib().b200fc_weight_unpack(self.h, dst_ptr, ld_bytes, stream))

    def group_scales(self, host_dst_ptr, ld_bytes, stream=None):
        """fp32 [N, ceil(K / INT4_GROUP)] dequant scales of 4-bit weights, into HOST memory."""
        check(lib().b200fc_weight_group_scales(self.h, host_dst_ptr, ld_bytes, stream))

    def export(self, stream=None):
        """Serialised form of the packed weights (bytearray); Weight.from_blob() rebuilds the object from it."""
        n = ctypes.c_size_t()
        check(lib().b200fc_weight_export_size(self.h, ctypes.byref(n)))
        buf = bytearray(n.value)
        view = (ctypes.c_char * n.value).from_buffer(buf)
        check(lib().b200fc_weight_export(self.h, ctypes.addressof(view), n.value, stream))
        del view
        return buf

    @classmethod
    def from_blob(cls, blob, stream=None):
        """blob: bytes-like object written by export() (e.g. read back from a file)."""
        raw = bytes(blob) if not isinstance(blob, (bytes, bytearray)) else blob
        src = (ctypes.c_char * len(raw)).from_buffer_copy(raw)
        h = c_void_p()
        check(lib().b200fc_weight_import(ctypes.addressof(src), len(raw), ctypes.byref(h), stream))
        self = cls.__new__(cls)
        self.h = h
        info = self.info()
        self.K, self.N = info["K"], info["N"]
        return self

    def matmul(self, A_ptr, dtypeA, M, K, lda_bytes, ep, n0=0, n1=None, stream=None):
        check(lib().b200fc_matmul(self.h, A_ptr, dtypeA, M, K, lda_bytes, n0, self.N if n1 is None else n1,
                                  ctypes.byref(ep), stream))

    def matmul_host(self, A_ptr, dtypeA, M, K, lda_bytes, ep, n0=0, n1=None, stream=None):
        check(lib().b200fc_matmul_host(self.h, A_ptr, dtypeA, M, K, lda_bytes, n0, self.N if n1 is None else n1,
                                       ctypes.byref(ep), stream))

    def close(self):
        if self.h:
            lib().b200fc_weight_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Mlp:
    """Fused Llama MLP (b200fc_mlp_t): AMX_MLP::MLP of the reference, optionally one tensor-parallel shard."""

    def __init__(self, gate_ptr, up_ptr, down_ptr, K, N, tp_rank=0, tp_size=1, stream=None):
        h = c_void_p()
        check(lib().b200fc_mlp_create(gate_ptr, up_ptr, down_ptr, K, N, tp_rank, tp_size, ctypes.byref(h), stream))
        self.h, self.K, self.N, self.tp_rank, self.tp_size = h, K, N, tp_rank, tp_size

    def reserve(self, max_M):
        check(lib().b200fc_mlp_reserve(self.h, max_M))

    def run(self, x_ptr, ldx_bytes, M, out_ptr, ldo_bytes, stream=None):
        check(lib().b200fc_mlp_run(self.h, x_ptr, ldx_bytes, M, out_ptr, ldo_bytes, stream))

    def run_partial(self, x_ptr, ldx_bytes, M, out_ptr, out_dtype, ldo_bytes, stream=None):
        check(lib().b200fc_mlp_run_partial(self.h, x_ptr, ldx_bytes, M, out_ptr, out_dtype, ldo_bytes, stream))

    def gate_up(self, x_ptr, ldx_bytes, M, stream=None):
        check(lib().b200fc_mlp_gate_up(self.h, x_ptr, ldx_bytes, M, stream))

    def down(self, M, out_ptr, out_dtype, ldo_bytes, stream=None):
        check(lib().b200fc_mlp_down(self.h, M, out_ptr, out_dtype, ldo_bytes, stream))

    def down_rows(self, row0, rows, out_ptr, out_dtype, ldo_bytes, stream=None):
        check(lib().b200fc_mlp_down_rows(self.h, row0, rows, out_ptr, out_dtype, ldo_bytes, stream))

    def down_reduce(self, M, multicast_ptr, out_dtype, ldo_bytes, stream=None):
        check(lib().b200fc_mlp_down_reduce(self.h, M, multicast_ptr, out_dtype, ldo_bytes, stream))

    def down_allreduce(self, M, ar, stream=None):
        """ar: capi.AllReduce; see b200fc_mlp_down_allreduce in include/b200fc.h."""
        check(lib().b200fc_mlp_down_allreduce(self.h, M, ctypes.byref(ar), stream))

    def run_host(self, x_ptr, ldx_bytes, M, out_ptr, ldo_bytes, stream=None):
        check(lib().b200fc_mlp_run_host(self.h, x_ptr, ldx_bytes, M, out_ptr, ldo_bytes, stream))

    def run_block(self, x_ptr, ldx_bytes, M, eps, out_ptr, ldo_bytes, norm_weight_ptr=None, add_residual=True, stream=None):
        """out = (x if add_residual else 0) + MLP(RMSNorm(x)); see b200fc_mlp_run_block in include/b200fc.h."""
        check(lib().b200fc_mlp_run_block(self.h, x_ptr, ldx_bytes, M, eps, norm_weight_ptr, 1 if add_residual else 0,
                                         out_ptr, ldo_bytes, stream))

    def run_decode_static(self, x_ptr, ldx_bytes, M, out_ptr, out_dtype, ldo_bytes, stream=None):
        """Allocation-free forward for 1 <= M <= 16; see b200fc_mlp_run_decode_static in include/b200fc.h."""
        check(lib().b200fc_mlp_run_decode_static(self.h, x_ptr, ldx_bytes, M, out_ptr, out_dtype, ldo_bytes, stream))

    def act_ptr(self):
        return lib().b200fc_mlp_act(self.h)

    def close(self):
        if self.h:
            lib().b200fc_mlp_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def matvec(A_ptr, dtype, M, K, lda_bytes, b_ptr, c_ptr, stream=None):
    check(lib().b200fc_matvec(A_ptr, dtype, M, K, lda_bytes, b_ptr, c_ptr, stream))


def matvec_host(A_ptr, dtype, M, K, lda_bytes, b_ptr, c_ptr, stream=None):
    check(lib().b200fc_matvec_host(A_ptr, dtype, M, K, lda_bytes, b_ptr, c_ptr, stream))


def memcpy(dst_ptr, src_ptr, nbytes, stream=None):
    check(lib().b200fc_memcpy(dst_ptr, src_ptr, nbytes, stream))


def rmsnorm(x_ptr, ldx_bytes, M, K, eps, out_ptr, ldo_bytes, weight_ptr=None, stream=None):
    check(lib().b200fc_rmsnorm(x_ptr, ldx_bytes, M, K, weight_ptr, eps, out_ptr, ldo_bytes, stream))


def decode_attention(desc, stream=None):
    """desc: capi.Attention; see b200fc_decode_attention in include/b200fc.h."""
    check(lib().b200fc_decode_attention(ctypes.byref(desc), stream))


def add_round_bf16(a_ptr, b_ptr, out_ptr, n, stream=None):
    check(lib().b200fc_add_round_bf16(a_ptr, b_ptr, out_ptr, n, stream))


def flush_l2(stream=None):
    check(lib().b200fc_flush_l2(stream))


def mlp_host_plan(M, K, N, capacity=4096):
    """row chunks of the host-buffer MLP call: (rows per gate/up launch, rows per down launch)"""
    g = (ctypes.c_int * capacity)(); d = (ctypes.c_int * capacity)()
    ng, nd = ctypes.c_int(), ctypes.c_int()
    check(lib().b200fc_mlp_host_plan(M, K, N, g, d, capacity, ctypes.byref(ng), ctypes.byref(nd)))
    return list(g[:ng.value]), list(d[:nd.value])
