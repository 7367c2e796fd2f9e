// C ABI of the b200fc library (declared in include/b200fc.h): argument checking, packed-weight and MLP objects,
// dispatch between the decode (gemv.cu) and prefill (gemm_tc.cu) kernels, host-buffer convenience entry points.
#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <new>
#include "common.cuh"

namespace b200fc {

// ---- error / bookkeeping --------------------------------------------------------------------------------------------
static thread_local char g_err[512] = "";
static std::atomic<long long> g_launches{0};

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
int cuda_fail(cudaError_t e, const char* what) {
    set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return e == cudaErrorMemoryAllocation ? B200FC_ERR_NOMEM : B200FC_ERR_CUDA;
}
void count_launch(int n) { g_launches += n; }

static std::atomic<int> g_sm_limit{0};
int sm_limit() { return g_sm_limit.load(); }

static std::atomic<unsigned long long> g_wait_limit_ns{2000000000ull};
unsigned long long wait_limit_ns() { return g_wait_limit_ns.load(); }

static std::mutex g_mu;
static std::map<int, int*> g_status;  // per device

// The status word is part of the library image (zero when a device loads it), so no call ever has to allocate it;
// host code needs its device address, looked up once per device.
static __device__ int g_status_word;

int* kernel_status_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_status.find(dev);
    if (it != g_status.end()) return it->second;
    int* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, g_status_word) != cudaSuccess || !p) { cudaGetLastError(); return nullptr; }
    g_status[dev] = p;
    return p;
}

int check_kernel_status(cudaStream_t s) {
    int* p = kernel_status_word();
    if (!p) { set_error("no kernel status word"); return B200FC_ERR_CUDA; }
    int v = 0;
    B200FC_CUDA(cudaMemcpyAsync(&v, p, sizeof(int), cudaMemcpyDeviceToHost, s));
    B200FC_CUDA(cudaStreamSynchronize(s));
    if (v != 0) {
        cudaMemsetAsync(p, 0, sizeof(int), s);
        set_error("a kernel gave up on a bounded wait (code %d)", v);
        return B200FC_ERR_KERNEL;
    }
    return B200FC_OK;
}

struct Scratch { void* p = nullptr; size_t bytes = 0; };
struct ScratchKey {
    int dev; cudaStream_t s; int slot;
    bool operator<(const ScratchKey& o) const {
        if (dev != o.dev) return dev < o.dev;
        if (s != o.s) return s < o.s;
        return slot < o.slot;
    }
};
static std::map<ScratchKey, Scratch> g_scratch;

int get_stream_scratch(size_t bytes, cudaStream_t s, int slot, void** out) {
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(g_mu);
    Scratch& sc = g_scratch[ScratchKey{dev, s, slot}];
    if (sc.bytes < bytes) {
        if (sc.p) { cudaStreamSynchronize(s); cudaFree(sc.p); sc.p = nullptr; sc.bytes = 0; }
        B200FC_CUDA(cudaMalloc(&sc.p, bytes));
        sc.bytes = bytes;
    }
    *out = sc.p;
    return B200FC_OK;
}

static int get_scratch(size_t bytes, cudaStream_t s, void** out) { return get_stream_scratch(bytes, s, 0, out); }

// Scratch of the decode kernel (fixed size, counters zero between launches), one per (device, stream).  A stream that
// first shows up while it is being captured into a CUDA graph cannot allocate (cudaMalloc is refused during capture),
// so the first call on a device also sets aside a few spare buffers that such streams take over.
static std::map<ScratchKey, void*> g_gemv_scratch;
static std::map<int, std::vector<void*>> g_gemv_spare;
constexpr int kGemvSpareBuffers = 8;

int get_gemv_scratch(cudaStream_t s, void** out) {
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(g_mu);
    const ScratchKey key{dev, s, 2};
    auto it = g_gemv_scratch.find(key);
    if (it != g_gemv_scratch.end()) { *out = it->second; return B200FC_OK; }
    const size_t bytes = gemv_scratch_bytes();
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cap) != cudaSuccess) { cudaGetLastError(); cap = cudaStreamCaptureStatusNone; }
    std::vector<void*>& spare = g_gemv_spare[dev];
    void* p = nullptr;
    if (cap != cudaStreamCaptureStatusNone) {
        if (spare.empty()) {
            set_error("decode kernel: no scratch for this stream and none can be allocated while it is being captured; "
                      "run one decode-shaped call on the device (any stream) before capturing");
            return B200FC_ERR_UNSUPPORTED;
        }
        p = spare.back();
        spare.pop_back();
    } else {
        const bool first_on_device = g_gemv_scratch.empty() && spare.empty();
        B200FC_CUDA(cudaMalloc(&p, bytes));
        B200FC_CUDA(cudaMemsetAsync(p, 0, bytes, s));
        if (first_on_device || spare.size() < 2) {
            // (re)fill the spare set; zeroed with a synchronous memset, whoever takes one over finds it ready
            while ((int)spare.size() < kGemvSpareBuffers) {
                void* q = nullptr;
                if (cudaMalloc(&q, bytes) != cudaSuccess) { cudaGetLastError(); break; }
                if (cudaMemset(q, 0, bytes) != cudaSuccess) { cudaGetLastError(); cudaFree(q); break; }
                spare.push_back(q);
            }
        }
    }
    g_gemv_scratch[key] = p;
    *out = p;
    return B200FC_OK;
}

static int grow(void** p, size_t* have, size_t need, cudaStream_t s) {
    if (*have >= need) return B200FC_OK;
    if (*p) { cudaStreamSynchronize(s); cudaFree(*p); *p = nullptr; *have = 0; }
    B200FC_CUDA(cudaMalloc(p, need));
    *have = need;
    return B200FC_OK;
}

static int elem_size(int dtype) {
    switch (dtype) {
        case B200FC_BF16: return 2;
        case B200FC_S8: case B200FC_U8: return 1;
        case B200FC_F32: case B200FC_S32: return 4;
    }
    return 0;
}

static bool is_device_ptr(const void* p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

static int round_up(int v, int m) { return (v + m - 1) / m * m; }

static int alloc_weight(Weight& w, int K, int N, int dtype) {
    w.K = K; w.N = N; w.dtype = dtype;
    w.N_pad = round_up(N, kRowPad);
    if (dtype == B200FC_S4) {
        w.K_pad = round_up(K, 2 * kKPadBytes);
        B200FC_CUDA(cudaMalloc(&w.data, w.data_bytes()));
        B200FC_CUDA(cudaMalloc(&w.scale_grp, w.scale_grp_floats() * sizeof(float)));
        return B200FC_OK;
    }
    const int es = elem_size(dtype);
    w.K_pad = round_up(K * es, kKPadBytes) / es;
    B200FC_CUDA(cudaMalloc(&w.data, w.data_bytes()));
    return B200FC_OK;
}

static void free_weight(Weight* w) {
    if (!w) return;
    cudaFree(w->data); cudaFree(w->scale_per_oc); cudaFree(w->scale_grp);
    cudaFree(w->stage_A); cudaFree(w->stage_C); cudaFree(w->stage_vec);
}

// Makes [rows, row_bytes] of a host or device matrix available on the device.  Device sources are used in place.
struct DevSrc {
    const void* p = nullptr; int64_t ld = 0; void* owned = nullptr;
    ~DevSrc() { if (owned) cudaFree(owned); }
};
static int to_device(const void* src, int64_t ld, int rows, size_t row_bytes, cudaStream_t s, DevSrc& out) {
    if (is_device_ptr(src)) { out.p = src; out.ld = ld; return B200FC_OK; }
    size_t pitch = (row_bytes + 15) / 16 * 16;
    B200FC_CUDA(cudaMalloc(&out.owned, pitch * (size_t)rows));
    B200FC_CUDA(cudaMemcpy2DAsync(out.owned, pitch, src, (size_t)ld, row_bytes, (size_t)rows, cudaMemcpyHostToDevice, s));
    out.p = out.owned; out.ld = (int64_t)pitch;
    return B200FC_OK;
}

static thread_local int g_mc_reduce = 0;  // set around one matmul_device call by mlp_down_device

static int validate_epilogue(const b200fc_epilogue_t* ep, bool int_acc) {
    if (!ep || !ep->C) { set_error("epilogue / C is null"); return B200FC_ERR_INVALID; }
    const int s = ep->steps;
    if (s & ~31) { set_error("unknown post-op bits 0x%x", s); return B200FC_ERR_INVALID; }
    if (s & B200FC_STEP_SILU_MUL) {
        if (s != B200FC_STEP_SILU_MUL || ep->out_dtype != B200FC_BF16 || int_acc) {
            set_error("SILU_MUL excludes the other steps and needs a bf16 GEMM with bf16 output");
            return B200FC_ERR_INVALID;
        }
    }
    if ((s & B200FC_STEP_BIAS) && !ep->bias) { set_error("STEP_BIAS without a bias pointer"); return B200FC_ERR_INVALID; }
    if (ep->out_dtype == B200FC_S32) {
        if (!int_acc || s != 0) { set_error("raw int32 output needs an 8-bit GEMM and no post-op"); return B200FC_ERR_INVALID; }
    } else if (ep->out_dtype != B200FC_F32 && ep->out_dtype != B200FC_BF16 && ep->out_dtype != B200FC_S8) {
        set_error("out_dtype must be f32, bf16, s8 (or s32 for raw accumulators)");
        return B200FC_ERR_INVALID;
    }
    return B200FC_OK;
}

int matmul_device(const Weight& w, Weight* w_mut, const void* A, int dtypeA, int M, int K, int64_t lda, int n0,
                  int n1, const b200fc_epilogue_t* ep_in, cudaStream_t s, void* gemv_scratch, const void* residual,
                  int64_t ld_res) {
    if (M < 0 || K != w.K) { set_error("matmul: K=%d does not match the packed weights (K=%d) or M<0", K, w.K); return B200FC_ERR_INVALID; }
    if (n0 < 0 || n1 > w.N || n0 > n1) { set_error("matmul: column range [%d,%d) outside [0,%d)", n0, n1, w.N); return B200FC_ERR_INVALID; }
    const bool a8 = dtypeA == B200FC_S8 || dtypeA == B200FC_U8;
    if (!a8 && dtypeA != B200FC_BF16) { set_error("matmul: dtypeA must be bf16, s8 or u8"); return B200FC_ERR_INVALID; }
    if (a8 && (w.dtype == B200FC_BF16 || w.compressed)) { set_error("matmul: 8-bit activations need plain 8-bit weights"); return B200FC_ERR_INVALID; }
    if (!a8 && w.dtype != B200FC_BF16 && !w.compressed) { set_error("matmul: bf16 activations need bf16 or compressed weights"); return B200FC_ERR_INVALID; }
    int rc = validate_epilogue(ep_in, a8);
    if (rc) return rc;
    if (lda < (int64_t)K * elem_size(dtypeA)) { set_error("matmul: lda smaller than a row"); return B200FC_ERR_INVALID; }
    if (M == 0 || n0 == n1) return B200FC_OK;

    Epilogue ep;
    ep.steps = ep_in->steps; ep.out_dtype = ep_in->out_dtype; ep.C = ep_in->C; ep.ldc = ep_in->ldc_bytes;
    ep.bias = ep_in->bias; ep.deq_scale = ep_in->deq_scale; ep.deq_per_oc = ep_in->deq_scale_per_oc;
    ep.q_scale = ep_in->q_scale; ep.q_per_oc = ep_in->q_scale_per_oc;
    ep.mc_reduce = g_mc_reduce;
    if (residual) {
        if ((ep.steps & B200FC_STEP_SILU_MUL) || (ep.out_dtype != B200FC_BF16 && ep.out_dtype != B200FC_F32) || g_mc_reduce) {
            set_error("matmul: a residual needs a bf16 or fp32 output without SILU_MUL");
            return B200FC_ERR_INVALID;
        }
        ep.residual = residual; ep.ld_res = ld_res;
    }
    if (ep.mc_reduce && M <= 16) { set_error("multicast-reduce output needs the tensor-core path (M > 16)"); return B200FC_ERR_UNSUPPORTED; }
    if (w.compressed) {
        if (!(ep.steps & B200FC_STEP_DEQUANT)) { set_error("matmul: compressed weights need STEP_DEQUANT"); return B200FC_ERR_INVALID; }
        ep.deq_scale = w.deq_scale;          // the weight's scale replaces the caller's (kernels_amx.hpp:1379)
        ep.deq_per_oc = w.scale_per_oc;
        if (w.dtype == B200FC_S4 && (n0 % 128)) { set_error("matmul: 4-bit weights need n0 to be a multiple of 128"); return B200FC_ERR_INVALID; }
    }
    if ((ep.steps & B200FC_STEP_SILU_MUL) && ((n0 % 32) || ((n1 - n0) % 32))) {
        set_error("matmul: SILU_MUL needs n0 and n1 multiples of 32");
        return B200FC_ERR_INVALID;
    }

    if (!a8 && M <= 16) return launch_gemv_tma(w, A, M, K, lda, n0, n1, ep, s, gemv_scratch);

    // tensor-core path: TMA needs a 16-byte aligned base and leading dimension
    const void* A_use = A;
    int64_t lda_use = lda;
    if (((uintptr_t)A & 15) || (lda & 15)) {
        const int es = elem_size(dtypeA);
        int64_t ld2 = round_up(K * es, 16);
        void* buf = nullptr;
        rc = get_scratch((size_t)ld2 * M, s, &buf);
        if (rc) return rc;
        rc = launch_copy2d(A, lda, buf, ld2, M, K * es, (int)ld2, s);
        if (rc) return rc;
        A_use = buf; lda_use = ld2;
    }
    if (w.compressed) {
        // M > 16 with compressed weights.  The reference decompresses 16 weight rows at a time into a reused
        // buffer right before the tile product (kernels_amx.hpp:1443-1514); here a block of weight rows is widened to
        // bf16 (exact for int8; 4-bit values are multiplied by their group scale and rounded to bf16, the one place
        // where the group scale cannot wait for the epilogue) into a per-stream scratch of at most 32 MB — small enough to stay in the 126 MB L2 until the
        // GEMM over those rows, launched right behind it, has read it — so HBM sees the int8 bytes only and no second
        // copy of the matrix is kept.
        (void)w_mut;
        const size_t row_bytes = (size_t)w.K_pad * 2;
        int blk = (int)(((size_t)32 << 20) / row_bytes) / kRowPad * kRowPad;
        if (blk < kRowPad) blk = kRowPad;
        const int r_lo = n0 / kRowPad * kRowPad;                  // packed rows are padded to kRowPad
        void* wide = nullptr;
        rc = get_stream_scratch((size_t)blk * row_bytes, s, 3, &wide);
        if (rc) return rc;
        for (int r0 = r_lo; r0 < n1; r0 += blk) {
            const int rows = (w.N_pad - r0 < blk) ? (w.N_pad - r0) : blk;
            const int c0 = r0 > n0 ? r0 : n0, c1 = (r0 + rows < n1) ? (r0 + rows) : n1;
            rc = launch_dequant_bf16(w, r0, rows, wide, w.K_pad, s);
            if (rc) return rc;
            // the block is addressed as a weight matrix whose row 0 is packed row r0: shift the column range and the
            // per-column arrays of the epilogue accordingly
            Epilogue e2 = ep;
            e2.C = (char*)ep.C + (long long)r0 * (ep.out_dtype == B200FC_F32 ? 4 : (ep.out_dtype == B200FC_BF16 ? 2 : 1));
            if (e2.bias) e2.bias += r0;
            if (e2.deq_per_oc) e2.deq_per_oc += r0;
            if (e2.q_per_oc) e2.q_per_oc += r0;
            if (e2.residual) e2.residual = (const char*)e2.residual + (long long)r0 * 2;
            rc = launch_gemm_tc(wide, B200FC_BF16, w.K_pad, rows, A_use, B200FC_BF16, M, K, lda_use, c0 - r0, c1 - r0, e2, s);
            if (rc) return rc;
        }
        return B200FC_OK;
    }
    return launch_gemm_tc(w.data, w.dtype, w.K_pad, w.N_pad, A_use, dtypeA, M, K, lda_use, n0, n1, ep, s);
}


static int mlp_gate_up_device(Mlp& m, const void* x, int64_t ldx, int M, cudaStream_t s) {
    if (M < 0) { set_error("mlp: M < 0"); return B200FC_ERR_INVALID; }
    if (M == 0) return B200FC_OK;
    int rc = grow(&m.act, &m.act_bytes, (size_t)M * m.Ns * 2, s);
    if (rc) return rc;
    m.act_rows = M;
    b200fc_epilogue_t e1 = {};
    e1.steps = B200FC_STEP_SILU_MUL; e1.out_dtype = B200FC_BF16; e1.C = m.act; e1.ldc_bytes = (int64_t)m.Ns * 2;
    return matmul_device(m.gate_up, nullptr, x, B200FC_BF16, M, m.K, ldx, 0, 2 * m.Ns, &e1, s);
}

static int mlp_down_device(Mlp& m, int M, void* out, int out_dtype, int64_t ldo, cudaStream_t s, int mc_reduce = 0,
                           int row0 = 0) {
    if (M < 0 || row0 < 0 || row0 + M > m.act_rows) { set_error("mlp_down: rows [%d, %d) outside the activation of the last gate_up (%d rows)", row0, row0 + M, m.act_rows); return B200FC_ERR_INVALID; }
    if (M == 0) return B200FC_OK;
    b200fc_epilogue_t e2 = {};
    e2.steps = 0; e2.out_dtype = out_dtype; e2.C = out; e2.ldc_bytes = ldo;
    g_mc_reduce = mc_reduce;
    const char* act = (const char*)m.act + (size_t)row0 * m.Ns * 2;
    int rc = matmul_device(m.down, nullptr, act, B200FC_BF16, M, m.Ns, (int64_t)m.Ns * 2, 0, m.K, &e2, s);
    g_mc_reduce = 0;
    return rc;
}

// Decode-shaped batches: both projections in one launch when the shape and the device allow it.  B200FC_ERR_UNSUPPORTED
// (no message) = not this time; the caller launches the two projections one after the other.
int mlp_decode_fused_device(const Mlp& m, const void* x, int64_t ldx, int M, void* act, void* out, int out_dtype,
                            int64_t ldo, cudaStream_t s, void* gemv_scratch, const void* residual, int64_t ld_res) {
    if (M < 1 || M > 16 || (out_dtype != B200FC_BF16 && out_dtype != B200FC_F32)) return B200FC_ERR_UNSUPPORTED;
    if (ldx < (int64_t)m.K * 2) { set_error("mlp: ldx smaller than a row"); return B200FC_ERR_INVALID; }
    Epilogue ep = {};
    ep.steps = 0; ep.out_dtype = out_dtype; ep.C = out; ep.ldc = ldo;
    ep.deq_scale = 1.0f; ep.q_scale = 1.0f;
    ep.residual = residual; ep.ld_res = ld_res;
    return launch_mlp_decode_fused(m.gate_up, m.down, x, ldx, M, m.K, m.Ns, act, ep, s, gemv_scratch);
}

static int mlp_run_device(Mlp& m, const void* x, int64_t ldx, int M, void* out, int out_dtype, int64_t ldo, cudaStream_t s) {
    if (M >= 1 && M <= 16) {
        int rc = grow(&m.act, &m.act_bytes, (size_t)M * m.Ns * 2, s);
        if (rc) return rc;
        rc = mlp_decode_fused_device(m, x, ldx, M, m.act, out, out_dtype, ldo, s, nullptr, nullptr, 0);
        if (rc != B200FC_ERR_UNSUPPORTED) {
            if (!rc) m.act_rows = M;
            return rc;
        }
    }
    int rc = mlp_gate_up_device(m, x, ldx, M, s);
    if (rc) return rc;
    return mlp_down_device(m, M, out, out_dtype, ldo, s);
}

}  // namespace b200fc

using namespace b200fc;


extern "C" {

const char* b200fc_last_error(void) { return g_err; }
const char* b200fc_version(void) { return "b200fc 0.1 (sm_100a)"; }
int64_t b200fc_launch_count(void) { return (int64_t)g_launches.load(); }

int b200fc_set_sm_limit(int sms) {
    if (sms < 0) { set_error("set_sm_limit: negative"); return B200FC_ERR_INVALID; }
    g_sm_limit = sms;
    return B200FC_OK;
}

int b200fc_set_decode_ctas_per_sm(int n) {
    if (n < 0 || n > 2) { set_error("set_decode_ctas_per_sm: 0 (default), 1 or 2"); return B200FC_ERR_INVALID; }
    set_decode_ctas_per_sm(n);
    return B200FC_OK;
}

int b200fc_sync_check(void* stream) { return check_kernel_status((cudaStream_t)stream); }

int b200fc_set_wait_limit_ns(uint64_t ns) {
    if (ns < 1000) { set_error("set_wait_limit_ns: limit below one microsecond"); return B200FC_ERR_INVALID; }
    g_wait_limit_ns = ns;
    return B200FC_OK;
}

int b200fc_weight_pack(const void* B, int dtypeB, int K, int N, int64_t ldb, int transposeB, int pack_mode,
                       const float* scales, b200fc_weight_t** out, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!B || !out || K <= 0 || N <= 0) { set_error("weight_pack: null pointer or empty shape"); return B200FC_ERR_INVALID; }
    const int es = elem_size(dtypeB);
    if (dtypeB != B200FC_BF16 && dtypeB != B200FC_S8 && dtypeB != B200FC_U8) { set_error("weight_pack: dtypeB must be bf16, s8 or u8"); return B200FC_ERR_INVALID; }
    const int rows = transposeB ? N : K, cols = transposeB ? K : N;
    if (ldb < (int64_t)cols * es) { set_error("weight_pack: ldb smaller than a row"); return B200FC_ERR_INVALID; }
    if (pack_mode == B200FC_PACK_QUANT_TENSOR && dtypeB != B200FC_BF16) { set_error("weight_pack: QUANT_TENSOR needs bf16 weights"); return B200FC_ERR_INVALID; }
    if (pack_mode == B200FC_PACK_INT8_CHANNEL && (dtypeB != B200FC_S8 || !scales)) { set_error("weight_pack: INT8_CHANNEL needs s8 weights and scales"); return B200FC_ERR_INVALID; }
    if (pack_mode == B200FC_PACK_INT4_GROUP && dtypeB != B200FC_BF16) { set_error("weight_pack: INT4_GROUP needs bf16 weights"); return B200FC_ERR_INVALID; }
    if (pack_mode < 0 || pack_mode > 3) { set_error("weight_pack: unknown pack mode"); return B200FC_ERR_INVALID; }

    b200fc_weight_t* h = new (std::nothrow) b200fc_weight_t;
    if (!h) { set_error("out of host memory"); return B200FC_ERR_NOMEM; }
    Weight& w = h->w;
    int rc;
    {
        DevSrc src;
        rc = to_device(B, ldb, rows, (size_t)cols * es, s, src);
        if (!rc) rc = alloc_weight(w, K, N, pack_mode == B200FC_PACK_QUANT_TENSOR ? B200FC_S8 : (pack_mode == B200FC_PACK_INT4_GROUP ? B200FC_S4 : dtypeB));
        if (!rc) {
            if (pack_mode == B200FC_PACK_INT4_GROUP) {
                // two passes: the bf16 matrix in packed row order (zero padded), then one warp per group of 128 K
                Weight wide;
                wide.K = K; wide.N = N; wide.dtype = B200FC_BF16; wide.K_pad = w.K_pad; wide.N_pad = w.N_pad;
                if (cudaMalloc(&wide.data, wide.data_bytes()) != cudaSuccess) rc = B200FC_ERR_NOMEM;
                if (!rc) rc = launch_pack(src.p, B200FC_BF16, K, N, src.ld, transposeB, wide, false, s);
                if (!rc) rc = launch_quant4(wide.data, w, s);
                if (!rc && cudaStreamSynchronize(s) != cudaSuccess) rc = B200FC_ERR_CUDA;
                cudaFree(wide.data);
                w.compressed = true;
                w.deq_scale = 1.0f;
            } else if (pack_mode == B200FC_PACK_QUANT_TENSOR) {
                float* absmax = nullptr;
                rc = cudaMalloc(&absmax, sizeof(float)) == cudaSuccess ? 0 : B200FC_ERR_NOMEM;
                if (!rc && scales) {  // caller-supplied absmax (e.g. of a larger matrix this one is a slice of)
                    if (cudaMemcpyAsync(absmax, scales, sizeof(float), cudaMemcpyDefault, s) != cudaSuccess) rc = B200FC_ERR_CUDA;
                } else if (!rc) {
                    rc = launch_absmax(src.p, rows, cols, src.ld, absmax, s);
                }
                if (!rc) rc = launch_quant_pack(src.p, K, N, src.ld, transposeB, w, absmax, s);
                float mx = 0.0f;
                if (!rc && cudaMemcpyAsync(&mx, absmax, sizeof(float), cudaMemcpyDeviceToHost, s) != cudaSuccess) rc = B200FC_ERR_CUDA;
                if (!rc && cudaStreamSynchronize(s) != cudaSuccess) rc = B200FC_ERR_CUDA;
                cudaFree(absmax);
                w.compressed = true;
                w.deq_scale = mx / 127;  // dequant_scale_B = max / 127 (kernels_amx.hpp:1373)
            } else {
                rc = launch_pack(src.p, dtypeB, K, N, src.ld, transposeB, w, pack_mode == B200FC_PACK_INT8_CHANNEL, s);
                if (!rc && pack_mode == B200FC_PACK_INT8_CHANNEL) {
                    w.compressed = true;
                    w.deq_scale = 1.0f;
                    if (cudaMalloc(&w.scale_per_oc, sizeof(float) * w.N_pad) != cudaSuccess) rc = B200FC_ERR_NOMEM;
                    if (!rc) cudaMemsetAsync(w.scale_per_oc, 0, sizeof(float) * w.N_pad, s);
                    if (!rc && cudaMemcpyAsync(w.scale_per_oc, scales, sizeof(float) * N, cudaMemcpyDefault, s) != cudaSuccess) rc = B200FC_ERR_CUDA;
                }
            }
        }
        if (!rc && cudaStreamSynchronize(s) != cudaSuccess) rc = B200FC_ERR_CUDA;  // the staged source dies with `src`
    }
    if (rc) {
        if (rc == B200FC_ERR_NOMEM) set_error("weight_pack: out of device memory");
        else if (rc == B200FC_ERR_CUDA && !g_err[0]) set_error("weight_pack: CUDA failure: %s", cudaGetErrorString(cudaGetLastError()));
        free_weight(&w); delete h; return rc;
    }
    *out = h;
    return B200FC_OK;
}

int b200fc_weight_free(b200fc_weight_t* w) {
    if (!w) return B200FC_OK;
    free_weight(&w->w);
    delete w;
    return B200FC_OK;
}

int b200fc_weight_info(const b200fc_weight_t* w, int* K, int* N, int* dtype, int* compressed, float* deq_scale) {
    if (!w) { set_error("weight_info: null handle"); return B200FC_ERR_INVALID; }
    if (K) *K = w->w.K;
    if (N) *N = w->w.N;
    if (dtype) *dtype = w->w.dtype;
    if (compressed) *compressed = w->w.compressed ? 1 : 0;
    if (deq_scale) *deq_scale = w->w.deq_scale;
    return B200FC_OK;
}

int b200fc_weight_unpack(const b200fc_weight_t* h, void* dst, int64_t ld_bytes, void* stream) {
    if (!h || !dst) { set_error("weight_unpack: null pointer"); return B200FC_ERR_INVALID; }
    const Weight& w = h->w;
    const int es = elem_size(w.dtype);
    cudaStream_t s = (cudaStream_t)stream;
    if (w.dtype == B200FC_S4) {
        void* tmp = nullptr;
        B200FC_CUDA(cudaMalloc(&tmp, (size_t)w.N * w.K));
        int rc = launch_unpack4(w, tmp, w.K, s);
        cudaError_t e = rc ? cudaSuccess : cudaMemcpy2DAsync(dst, (size_t)ld_bytes, tmp, (size_t)w.K, (size_t)w.K, (size_t)w.N, cudaMemcpyDefault, s);
        cudaStreamSynchronize(s);
        cudaFree(tmp);
        if (rc) return rc;
        B200FC_CUDA(e);
        return B200FC_OK;
    }
    if (w.compressed) {  // stored offset-binary: hand back two's complement
        void* tmp = nullptr;
        B200FC_CUDA(cudaMalloc(&tmp, (size_t)w.N * w.K));
        int rc = launch_flip_copy2d(w.data, w.K_pad, tmp, w.K, w.N, w.K, s);
        cudaError_t e = rc ? cudaSuccess : cudaMemcpy2DAsync(dst, (size_t)ld_bytes, tmp, (size_t)w.K, (size_t)w.K, (size_t)w.N, cudaMemcpyDefault, s);
        cudaStreamSynchronize(s);
        cudaFree(tmp);
        if (rc) return rc;
        B200FC_CUDA(e);
        return B200FC_OK;
    }
    B200FC_CUDA(cudaMemcpy2DAsync(dst, (size_t)ld_bytes, w.data, (size_t)w.K_pad * es, (size_t)w.K * es, (size_t)w.N,
                                  cudaMemcpyDefault, s));
    B200FC_CUDA(cudaStreamSynchronize(s));
    return B200FC_OK;
}

int b200fc_weight_group_scales(const b200fc_weight_t* h, float* host_dst, int64_t ld_bytes, void* stream) {
    if (!h || !host_dst) { set_error("weight_group_scales: null pointer"); return B200FC_ERR_INVALID; }
    const Weight& w = h->w;
    if (w.dtype != B200FC_S4 || !w.scale_grp) { set_error("weight_group_scales: not a 4-bit weight"); return B200FC_ERR_INVALID; }
    const int groups = (w.K + B200FC_INT4_GROUP - 1) / B200FC_INT4_GROUP;
    if (ld_bytes < (int64_t)groups * 4) { set_error("weight_group_scales: ld smaller than a row"); return B200FC_ERR_INVALID; }
    std::vector<float> tmp(w.scale_grp_floats());
    cudaStream_t s = (cudaStream_t)stream;
    B200FC_CUDA(cudaMemcpyAsync(tmp.data(), w.scale_grp, tmp.size() * sizeof(float), cudaMemcpyDeviceToHost, s));
    B200FC_CUDA(cudaStreamSynchronize(s));
    const int spr = w.K_pad / 256;
    for (int n = 0; n < w.N; n++) {
        float* row = (float*)((char*)host_dst + (int64_t)n * ld_bytes);
        for (int j = 0; j < groups; j++)
            row[j] = tmp[((((size_t)(n >> 7) * spr) + (j >> 1)) * 2 + (j & 1)) * 128 + (n & 127)];
    }
    return B200FC_OK;
}

// ---- serialised packed weights ----------------------------------------------------------------------------------
namespace {
struct BlobHeader {           // 64 bytes, little endian
    char magic[8];            // "B2FCWGT1": the 1 is the packing version
    uint32_t header_bytes;    // 64
    int32_t dtype, K, N, K_pad, N_pad, compressed, has_scales;
    float deq_scale;
    uint32_t reserved;
    uint64_t data_bytes;      // N_pad * K_pad * element size
    uint64_t total_bytes;     // header + data + scales
};
static_assert(sizeof(BlobHeader) == 64, "blob header layout");
const char kBlobMagic[8] = {'B', '2', 'F', 'C', 'W', 'G', 'T', '1'};

uint64_t blob_scale_bytes(int has_scales, const Weight& w) {
    if (has_scales == 2) return (uint64_t)w.scale_grp_floats() * sizeof(float);
    return has_scales ? (uint64_t)w.N_pad * sizeof(float) : 0;
}

void fill_blob_header(const Weight& w, BlobHeader* hd) {
    memset(hd, 0, sizeof(*hd));
    memcpy(hd->magic, kBlobMagic, 8);
    hd->header_bytes = 64;
    hd->dtype = w.dtype; hd->K = w.K; hd->N = w.N; hd->K_pad = w.K_pad; hd->N_pad = w.N_pad;
    hd->compressed = w.compressed ? 1 : 0;
    hd->has_scales = w.scale_grp ? 2 : (w.scale_per_oc ? 1 : 0);   // 1: per output channel, 2: per group (4-bit weights)
    hd->deq_scale = w.deq_scale;
    hd->data_bytes = (uint64_t)w.data_bytes();
    hd->total_bytes = 64 + hd->data_bytes + blob_scale_bytes(hd->has_scales, w);
}
}  // namespace

int b200fc_weight_export_size(const b200fc_weight_t* h, size_t* bytes) {
    if (!h || !bytes) { set_error("weight_export_size: null pointer"); return B200FC_ERR_INVALID; }
    BlobHeader hd;
    fill_blob_header(h->w, &hd);
    *bytes = (size_t)hd.total_bytes;
    return B200FC_OK;
}

int b200fc_weight_export(const b200fc_weight_t* h, void* host_dst, size_t capacity, void* stream) {
    if (!h || !host_dst) { set_error("weight_export: null pointer"); return B200FC_ERR_INVALID; }
    const Weight& w = h->w;
    BlobHeader hd;
    fill_blob_header(w, &hd);
    if (capacity < hd.total_bytes) {
        set_error("weight_export: buffer of %zu bytes, %llu needed", capacity, (unsigned long long)hd.total_bytes);
        return B200FC_ERR_INVALID;
    }
    cudaStream_t s = (cudaStream_t)stream;
    char* dst = (char*)host_dst;
    memcpy(dst, &hd, sizeof(hd));
    B200FC_CUDA(cudaMemcpyAsync(dst + 64, w.data, (size_t)hd.data_bytes, cudaMemcpyDeviceToHost, s));
    if (hd.has_scales)
        B200FC_CUDA(cudaMemcpyAsync(dst + 64 + hd.data_bytes, hd.has_scales == 2 ? w.scale_grp : w.scale_per_oc,
                                    (size_t)blob_scale_bytes(hd.has_scales, w), cudaMemcpyDeviceToHost, s));
    B200FC_CUDA(cudaStreamSynchronize(s));
    return B200FC_OK;
}

int b200fc_weight_import(const void* host_src, size_t bytes, b200fc_weight_t** out, void* stream) {
    if (!host_src || !out) { set_error("weight_import: null pointer"); return B200FC_ERR_INVALID; }
    if (bytes < sizeof(BlobHeader)) { set_error("weight_import: %zu bytes is shorter than a header", bytes); return B200FC_ERR_INVALID; }
    BlobHeader hd;
    memcpy(&hd, host_src, sizeof(hd));
    if (memcmp(hd.magic, kBlobMagic, 8) != 0 || hd.header_bytes != 64) {
        set_error("weight_import: not a packed-weight blob of this library version");
        return B200FC_ERR_INVALID;
    }
    const bool known = hd.dtype == B200FC_BF16 || hd.dtype == B200FC_S8 || hd.dtype == B200FC_U8 || hd.dtype == B200FC_S4;
    if (!known || hd.K <= 0 || hd.N <= 0) { set_error("weight_import: bad dtype or shape in the header"); return B200FC_ERR_INVALID; }
    Weight shape;   // what alloc_weight would make of (K, N, dtype), without allocating
    shape.K = hd.K; shape.N = hd.N; shape.dtype = hd.dtype;
    shape.N_pad = round_up(hd.N, kRowPad);
    shape.K_pad = hd.dtype == B200FC_S4 ? round_up(hd.K, 2 * kKPadBytes) : round_up(hd.K * elem_size(hd.dtype), kKPadBytes) / elem_size(hd.dtype);
    const int K_pad = shape.K_pad, N_pad = shape.N_pad;
    const uint64_t data_bytes = (uint64_t)shape.data_bytes();
    const bool scales_ok = hd.has_scales == 0 || (hd.has_scales == 1 && hd.dtype == B200FC_S8) || (hd.has_scales == 2 && hd.dtype == B200FC_S4);
    const uint64_t scale_bytes = scales_ok ? blob_scale_bytes(hd.has_scales, shape) : 0;
    const uint64_t total = 64 + data_bytes + scale_bytes;
    if (hd.K_pad != K_pad || hd.N_pad != N_pad || hd.data_bytes != data_bytes || hd.total_bytes != total || bytes < total ||
        (hd.compressed && hd.dtype != B200FC_S8 && hd.dtype != B200FC_S4) || (hd.has_scales && !hd.compressed) || !scales_ok ||
        (hd.dtype == B200FC_S4 && (hd.has_scales != 2 || !hd.compressed))) {
        set_error("weight_import: header does not describe a blob this library wrote (or the buffer is truncated)");
        return B200FC_ERR_INVALID;
    }
    b200fc_weight_t* h = new (std::nothrow) b200fc_weight_t;
    if (!h) { set_error("out of host memory"); return B200FC_ERR_NOMEM; }
    Weight& w = h->w;
    cudaStream_t s = (cudaStream_t)stream;
    const char* src = (const char*)host_src;
    int rc = alloc_weight(w, hd.K, hd.N, hd.dtype);
    if (!rc && cudaMemcpyAsync(w.data, src + 64, (size_t)data_bytes, cudaMemcpyHostToDevice, s) != cudaSuccess) rc = B200FC_ERR_CUDA;
    if (!rc && hd.has_scales == 1) {
        if (cudaMalloc(&w.scale_per_oc, (size_t)N_pad * sizeof(float)) != cudaSuccess) rc = B200FC_ERR_NOMEM;
        if (!rc && cudaMemcpyAsync(w.scale_per_oc, src + 64 + data_bytes, (size_t)N_pad * sizeof(float), cudaMemcpyHostToDevice, s) != cudaSuccess)
            rc = B200FC_ERR_CUDA;
    }
    if (!rc && hd.has_scales == 2 &&
        cudaMemcpyAsync(w.scale_grp, src + 64 + data_bytes, (size_t)scale_bytes, cudaMemcpyHostToDevice, s) != cudaSuccess)
        rc = B200FC_ERR_CUDA;
    if (!rc && cudaStreamSynchronize(s) != cudaSuccess) rc = B200FC_ERR_CUDA;
    if (rc) {
        if (rc == B200FC_ERR_NOMEM) set_error("weight_import: out of device memory");
        else if (rc == B200FC_ERR_CUDA && !g_err[0]) set_error("weight_import: CUDA failure: %s", cudaGetErrorString(cudaGetLastError()));
        free_weight(&w); delete h; return rc;
    }
    w.compressed = hd.compressed != 0;
    w.deq_scale = hd.deq_scale;
    *out = h;
    return B200FC_OK;
}

int b200fc_matmul(const b200fc_weight_t* W, const void* A, int dtypeA, int M, int K, int64_t lda_bytes, int n0, int n1,
                  const b200fc_epilogue_t* ep, void* stream) {
    if (!W || !A) { set_error("matmul: null pointer"); return B200FC_ERR_INVALID; }
    return matmul_device(W->w, nullptr, A, dtypeA, M, K, lda_bytes, n0, n1, ep, (cudaStream_t)stream);
}

int b200fc_matmul_host(b200fc_weight_t* W, const void* A, int dtypeA, int M, int K, int64_t lda, int n0, int n1,
                       const b200fc_epilogue_t* ep, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!W || !A || !ep || !ep->C) { set_error("matmul_host: null pointer"); return B200FC_ERR_INVALID; }
    Weight& w = W->w;
    if (M <= 0 || n1 <= n0 || n0 < 0 || n1 > w.N) { set_error("matmul_host: empty or invalid range"); return B200FC_ERR_INVALID; }
    const int esA = elem_size(dtypeA), esC = elem_size(ep->out_dtype);
    if (!esA || !esC) { set_error("matmul_host: bad dtype"); return B200FC_ERR_INVALID; }
    const bool silu = (ep->steps & B200FC_STEP_SILU_MUL) != 0;
    const size_t rowA = (size_t)K * esA, ldA = (rowA + 15) / 16 * 16;
    const int out_cols = silu ? (n1 - n0) / 2 : (n1 - n0);
    const size_t rowC = (size_t)out_cols * esC, ldC = (rowC + 15) / 16 * 16;
    int rc = grow(&w.stage_A, &w.stage_A_bytes, ldA * M, s);
    if (!rc) rc = grow(&w.stage_C, &w.stage_C_bytes, ldC * M, s);
    size_t vec_floats = (size_t)n1 * 3;
    void* sv = w.stage_vec; size_t have = w.stage_vec_floats * sizeof(float);
    if (!rc) rc = grow(&sv, &have, vec_floats * sizeof(float), s);
    w.stage_vec = (float*)sv; w.stage_vec_floats = have / sizeof(float);
    if (rc) return rc;
    B200FC_CUDA(cudaMemcpy2DAsync(w.stage_A, ldA, A, (size_t)lda, rowA, (size_t)M, cudaMemcpyHostToDevice, s));
    b200fc_epilogue_t e = *ep;
    float* v = w.stage_vec;
    if (ep->bias) { B200FC_CUDA(cudaMemcpyAsync(v, ep->bias, sizeof(float) * n1, cudaMemcpyHostToDevice, s)); e.bias = v; }
    if (ep->deq_scale_per_oc) { B200FC_CUDA(cudaMemcpyAsync(v + n1, ep->deq_scale_per_oc, sizeof(float) * n1, cudaMemcpyHostToDevice, s)); e.deq_scale_per_oc = v + n1; }
    if (ep->q_scale_per_oc) { B200FC_CUDA(cudaMemcpyAsync(v + 2 * (size_t)n1, ep->q_scale_per_oc, sizeof(float) * n1, cudaMemcpyHostToDevice, s)); e.q_scale_per_oc = v + 2 * (size_t)n1; }
    // the kernels index C by the global column: shift the base so that column n0 lands at the start of the staging row
    const int64_t col0 = silu ? (int64_t)(n0 / 2) * esC : (int64_t)n0 * esC;
    e.C = (char*)w.stage_C - col0;
    e.ldc_bytes = (int64_t)ldC;
    rc = matmul_device(w, &w, w.stage_A, dtypeA, M, K, (int64_t)ldA, n0, n1, &e, s);
    if (rc) return rc;
    B200FC_CUDA(cudaMemcpy2DAsync((char*)ep->C + col0, (size_t)ep->ldc_bytes, w.stage_C, ldC, rowC, (size_t)M,
                                  cudaMemcpyDeviceToHost, s));
    return check_kernel_status(s);
}

int b200fc_matvec(const void* A, int dtype, int M, int K, int64_t lda, const void* b, void* c, void* stream) {
    if (!A || !b || !c || K <= 0 || M < 0) { set_error("matvec: null pointer or bad shape"); return B200FC_ERR_INVALID; }
    if (lda < (int64_t)K * elem_size(dtype)) { set_error("matvec: lda smaller than a row"); return B200FC_ERR_INVALID; }
    return launch_matvec(A, dtype, M, K, lda, b, c, (cudaStream_t)stream);
}

int b200fc_matvec_host(const void* A, int dtype, int M, int K, int64_t lda, const void* b, void* c, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!A || !b || !c || K <= 0 || M <= 0) { set_error("matvec_host: null pointer or bad shape"); return B200FC_ERR_INVALID; }
    const int es = elem_size(dtype);
    if (dtype != B200FC_BF16 && dtype != B200FC_S8) { set_error("matvec: dtype must be bf16 or s8"); return B200FC_ERR_INVALID; }
    const size_t row = (size_t)K * es, ld = (row + 15) / 16 * 16;
    void* buf = nullptr;
    int rc = get_scratch(ld * M + ld + (size_t)M * 4 + 64, s, &buf);
    if (rc) return rc;
    char* dA = (char*)buf; char* db = dA + ld * M; char* dc = db + ld;
    B200FC_CUDA(cudaMemcpy2DAsync(dA, ld, A, (size_t)lda, row, (size_t)M, cudaMemcpyHostToDevice, s));
    B200FC_CUDA(cudaMemcpyAsync(db, b, row, cudaMemcpyHostToDevice, s));
    rc = launch_matvec(dA, dtype, M, K, (int64_t)ld, db, dc, s);
    if (rc) return rc;
    B200FC_CUDA(cudaMemcpyAsync(c, dc, (size_t)M * 4, cudaMemcpyDeviceToHost, s));
    B200FC_CUDA(cudaStreamSynchronize(s));
    return B200FC_OK;
}

int b200fc_mlp_create(const void* gate, const void* up, const void* down, int K, int N, int tp_rank, int tp_size,
                      b200fc_mlp_t** out, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!gate || !up || !down || !out) { set_error("mlp_create: null pointer"); return B200FC_ERR_INVALID; }
    if (tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size || K <= 0 || N <= 0 || N % tp_size) { set_error("mlp_create: bad tensor-parallel split"); return B200FC_ERR_INVALID; }
    const int Ns = N / tp_size;
    if (K % 64 || Ns % 32) { set_error("mlp_create: need K %% 64 == 0 and (N / tp_size) %% 32 == 0"); return B200FC_ERR_INVALID; }
    b200fc_mlp_t* h = new (std::nothrow) b200fc_mlp_t;
    if (!h) { set_error("out of host memory"); return B200FC_ERR_NOMEM; }
    Mlp& m = h->m;
    m.K = K; m.N = N; m.Ns = Ns; m.tp_rank = tp_rank; m.tp_size = tp_size;
    int rc;
    {
        // this rank's rows of gate / up ([N, K]) and columns of down ([K, N])
        const char* g0 = (const char*)gate + (size_t)tp_rank * Ns * K * 2;
        const char* u0 = (const char*)up + (size_t)tp_rank * Ns * K * 2;
        const char* d0 = (const char*)down + (size_t)tp_rank * Ns * 2;
        DevSrc sg, su, sd;
        rc = to_device(g0, (int64_t)K * 2, Ns, (size_t)K * 2, s, sg);
        if (!rc) rc = to_device(u0, (int64_t)K * 2, Ns, (size_t)K * 2, s, su);
        if (!rc) rc = to_device(d0, (int64_t)N * 2, K, (size_t)Ns * 2, s, sd);
        if (!rc && sg.ld != su.ld) { set_error("mlp_create: gate and up must live in the same kind of memory"); rc = B200FC_ERR_INVALID; }
        if (!rc) rc = alloc_weight(m.gate_up, K, 2 * Ns, B200FC_BF16);
        if (!rc) rc = alloc_weight(m.down, Ns, K, B200FC_BF16);
        if (!rc) rc = launch_pack_gate_up(sg.p, su.p, sg.ld, K, Ns, m.gate_up, s);
        if (!rc) rc = launch_pack(sd.p, B200FC_BF16, Ns, K, sd.ld, 1, m.down, false, s);
        if (!rc && cudaStreamSynchronize(s) != cudaSuccess) { rc = cuda_fail(cudaGetLastError(), "mlp_create sync"); }
    }
    if (rc) { free_weight(&m.gate_up); free_weight(&m.down); delete h; return rc; }
    *out = h;
    return B200FC_OK;
}

int b200fc_mlp_free(b200fc_mlp_t* h) {
    if (!h) return B200FC_OK;
    free_weight(&h->m.gate_up); free_weight(&h->m.down);
    cudaFree(h->m.act); cudaFree(h->m.stage_x); cudaFree(h->m.stage_o);
    for (int i = 0; i < 3; i++) if (h->m.pipe_streams[i]) cudaStreamDestroy(h->m.pipe_streams[i]);
    if (h->m.ev_fork) cudaEventDestroy(h->m.ev_fork);
    if (h->m.ev_join) cudaEventDestroy(h->m.ev_join);
    for (cudaEvent_t e : h->m.ev_in) cudaEventDestroy(e);
    for (cudaEvent_t e : h->m.ev_out) cudaEventDestroy(e);
    delete h;
    return B200FC_OK;
}

int b200fc_mlp_reserve(b200fc_mlp_t* h, int max_M) {
    if (!h || max_M < 0) { set_error("mlp_reserve: bad argument"); return B200FC_ERR_INVALID; }
    return grow(&h->m.act, &h->m.act_bytes, (size_t)max_M * h->m.Ns * 2, 0);
}

int b200fc_mlp_run(b200fc_mlp_t* h, const void* x, int64_t ldx, int M, void* out, int64_t ldo, void* stream) {
    if (!h || !x || !out) { set_error("mlp_run: null pointer"); return B200FC_ERR_INVALID; }
    if (h->m.tp_size != 1) { set_error("mlp_run: tensor-parallel shard; use mlp_run_partial and sum over ranks"); return B200FC_ERR_INVALID; }
    return mlp_run_device(h->m, x, ldx, M, out, B200FC_BF16, ldo, (cudaStream_t)stream);
}

int b200fc_mlp_run_partial(b200fc_mlp_t* h, const void* x, int64_t ldx, int M, void* partial, int out_dtype, int64_t ldp,
                           void* stream) {
    if (!h || !x || !partial) { set_error("mlp_run_partial: null pointer"); return B200FC_ERR_INVALID; }
    if (out_dtype != B200FC_F32 && out_dtype != B200FC_BF16) { set_error("mlp_run_partial: out_dtype must be f32 or bf16"); return B200FC_ERR_INVALID; }
    return mlp_run_device(h->m, x, ldx, M, partial, out_dtype, ldp, (cudaStream_t)stream);
}

int b200fc_mlp_gate_up(b200fc_mlp_t* h, const void* x, int64_t ldx, int M, void* stream) {
    if (!h || !x) { set_error("mlp_gate_up: null pointer"); return B200FC_ERR_INVALID; }
    return mlp_gate_up_device(h->m, x, ldx, M, (cudaStream_t)stream);
}

int b200fc_mlp_down(b200fc_mlp_t* h, int M, void* out, int out_dtype, int64_t ldo, void* stream) {
    if (!h || !out) { set_error("mlp_down: null pointer"); return B200FC_ERR_INVALID; }
    if (out_dtype != B200FC_F32 && out_dtype != B200FC_BF16) { set_error("mlp_down: out_dtype must be f32 or bf16"); return B200FC_ERR_INVALID; }
    return mlp_down_device(h->m, M, out, out_dtype, ldo, (cudaStream_t)stream);
}

int b200fc_mlp_down_rows(b200fc_mlp_t* h, int row0, int rows, void* out, int out_dtype, int64_t ldo, void* stream) {
    if (!h || !out) { set_error("mlp_down_rows: null pointer"); return B200FC_ERR_INVALID; }
    if (out_dtype != B200FC_F32 && out_dtype != B200FC_BF16) { set_error("mlp_down_rows: out_dtype must be f32 or bf16"); return B200FC_ERR_INVALID; }
    return mlp_down_device(h->m, rows, out, out_dtype, ldo, (cudaStream_t)stream, 0, row0);
}

int b200fc_mlp_down_reduce(b200fc_mlp_t* h, int M, void* multicast_out, int out_dtype, int64_t ldo, void* stream) {
    if (!h || !multicast_out) { set_error("mlp_down_reduce: null pointer"); return B200FC_ERR_INVALID; }
    if (out_dtype != B200FC_F32 && out_dtype != B200FC_BF16) { set_error("mlp_down_reduce: out_dtype must be f32 or bf16"); return B200FC_ERR_INVALID; }
    if (M <= 16) { set_error("mlp_down_reduce: needs M > 16 (decode-shaped batches use mlp_run_partial + an all-reduce)"); return B200FC_ERR_UNSUPPORTED; }
    return mlp_down_device(h->m, M, multicast_out, out_dtype, ldo, (cudaStream_t)stream, 1);
}

int b200fc_mlp_down_allreduce(b200fc_mlp_t* h, int M, const b200fc_allreduce_t* ar, void* stream) {
    if (!h || !ar || !ar->partial_local || !ar->partial_mc || !ar->out_mc) { set_error("mlp_down_allreduce: null pointer"); return B200FC_ERR_INVALID; }
    Mlp& m = h->m;
    if (M <= 16) { set_error("mlp_down_allreduce: needs M > 16 (decode-shaped batches use mlp_run_partial + an all-reduce)"); return B200FC_ERR_UNSUPPORTED; }
    if (M > m.act_rows) { set_error("mlp_down_allreduce: no activation of %d rows (gate_up ran %d)", M, m.act_rows); return B200FC_ERR_INVALID; }
    AllReduceDesc d;
    d.world = ar->world; d.rank = ar->rank;
    d.partial_local = ar->partial_local; d.partial_mc = ar->partial_mc; d.out_mc = ar->out_mc;
    d.ld_bytes = ar->ld_bytes;
    for (int i = 0; i < 8; i++) {
        d.flags[i] = (i < ar->world) ? ar->flags[i] : nullptr;
        if (i < ar->world && !ar->flags[i]) { set_error("mlp_down_allreduce: missing counter array of rank %d", i); return B200FC_ERR_INVALID; }
    }
    d.max_tiles = ar->max_tiles; d.comm_sms = ar->comm_sms;
    return launch_gemm_tc_allreduce(m.down.data, m.down.K_pad, m.down.N_pad, m.act, M, m.Ns, (int64_t)m.Ns * 2, m.K, d,
                                    (cudaStream_t)stream);
}

// Row chunks of the host-buffer pipeline of b200fc_mlp_run_host: gu = rows per gate/up launch (each preceded by the
// host-to-device copy of its rows), dn = rows per down launch (each followed by the device-to-host copy of its rows);
// both lists sum to M.  The two lists are chosen independently: a handful of growing sequences (short chunks first,
// so that little of the first copy is exposed) for gate/up, the same sequences reversed and a halving sequence for
// down (short chunks last), each pair rated by a small model of the three engines — the copy engines at PCIe speed and
// the GEMMs as whole waves of 256 x 256 tiles over the CTA pairs, which is what makes a chunk of 7 x 256 rows of the
// Llama-70B down projection (224 tiles on 74 pairs) cost four waves instead of three.  The model only has to rank
// plans; measured on Llama-70B at M = 4096 its first choices are the measured first choices.
// B200FC_HOST_PLAN="a,b,c;d,e,f" (chunks in tiles of 256 rows; the last entry of each list takes what is left)
// replaces the choice, for experiments.
namespace {
constexpr int kPlanTile = 256;

struct PlanModel {
    double t_gu_wave, t_dn_wave;  // seconds per wave of tiles
    double h2d_tile, d2h_tile;    // seconds per 256 rows
    int cols_gu, cols_dn, pairs;
    int slabs_gu, slabs_dn;       // K of the two GEMMs in 64-element slabs
    // rounds of tiles a launch of `rows` row tiles x `cols` column tiles takes; a short ragged last round of a long-K
    // GEMM is split along K by the launcher (launch_gemm_tc) and costs well under a round
    double waves(int rows, int cols, int k_slabs) const {
        const long long tiles = (long long)rows * cols;
        const long long full = tiles / pairs, rem = tiles % pairs;
        if (rem == 0) return (double)full;
        if (full == 0 && tiles * 2 <= pairs && k_slabs >= 16) {  // few tiles: the launcher splits K over the idle pairs
            long long sp = std::min<long long>(std::min<long long>(8, pairs / tiles), k_slabs / 8);
            return 1.0 / (double)std::max<long long>(1, sp) + 0.35;  // (+ the slab round trip and the reduction kernel)
        }
        const bool split = full > 0 && rem * 4 <= pairs && k_slabs >= 96 && (rem / rows == 0 || rem % rows == 0);
        return (double)full + (split ? 0.45 : 1.0);
    }
    double run(const std::vector<int>& gu, const std::vector<int>& dn) const {
        const double copy_lat = 8e-6, launch_lat = 3e-6;
        double t_in = 0, t_cmp = 0, t_out = 0;
        size_t gi = 0;
        int done = 0, d0 = 0;
        for (size_t j = 0; j < dn.size(); j++) {
            const int d1 = d0 + dn[j];
            while (done < d1 && gi < gu.size()) {
                t_in += gu[gi] * h2d_tile + copy_lat;
                t_cmp = std::max(t_cmp, t_in) + waves(gu[gi], cols_gu, slabs_gu) * t_gu_wave + launch_lat;
                done += gu[gi++];
            }
            t_cmp += waves(dn[j], cols_dn, slabs_dn) * t_dn_wave + launch_lat;
            t_out = std::max(t_out, t_cmp) + dn[j] * d2h_tile + copy_lat;
            d0 = d1;
        }
        return t_out;
    }
};

// growing sequence: first, then each chunk `ratio` times the one before, at most `cap`, until `tiles` are covered
std::vector<int> growing(int tiles, int first, double ratio, int cap) {
    std::vector<int> v;
    int left = tiles;
    double cur = first;
    while (left > 0) {
        int c = std::min(left, std::min(cap, (int)(cur + 0.5)));
        if (c < 1) c = 1;
        v.push_back(c);
        left -= c;
        cur = std::min((double)cap, std::max(cur * ratio, cur));
    }
    if (v.size() > 1 && v.back() * 2 < v[v.size() - 2]) {  // a crumb at the end joins its neighbour
        v[v.size() - 2] += v.back();
        v.pop_back();
    }
    return v;
}
}  // namespace

static void host_plan(Mlp* cache, int K_, int Ns_, int M, std::vector<int>* gu, std::vector<int>* dn) {
    const int tile = kPlanTile;
    const int tiles = (M + tile - 1) / tile;
    auto finish = [&](std::vector<int>& v) {  // tiles -> rows, clipped to M
        int left = M;
        std::vector<int> r;
        for (size_t i = 0; i < v.size() && left > 0; i++) {
            int rows = (i + 1 == v.size()) ? left : (int)std::min<long long>(left, (long long)v[i] * tile);
            if (rows > 0) r.push_back(rows);
            left -= rows;
        }
        if (left > 0) r.push_back(left);
        v.swap(r);
    };
    std::vector<int> g, d;
    const char* env = getenv("B200FC_HOST_PLAN");
    if (env && *env) {
        std::vector<int>* cur = &g;
        int val = 0; bool have = false;
        for (const char* c = env;; c++) {
            if (*c >= '0' && *c <= '9') { val = val * 10 + (*c - '0'); have = true; continue; }
            if (have && val > 0) cur->push_back(val);
            val = 0; have = false;
            if (*c == ';') cur = &d;
            if (!*c) break;
        }
        if (!g.empty() && !d.empty()) {
            finish(g); finish(d);
            gu->swap(g); dn->swap(d);
            return;
        }
    }
    if (cache && cache->plan_M == M && !cache->plan_gu.empty()) { *gu = cache->plan_gu; *dn = cache->plan_dn; return; }
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        cudaGetLastError();   // no device (a host-only process asking for the plan): a B200's 148 SMs
        sms = 148;
    }
    PlanModel pm;
    pm.pairs = std::max(1, sms / 2);
    const double pair_rate = 1.35e15 / 74.0;  // flop/s of one CTA pair in a long launch
    pm.cols_gu = (2 * Ns_ + 255) / 256;
    pm.cols_dn = (K_ + 255) / 256;
    pm.slabs_gu = (K_ + 63) / 64;
    pm.slabs_dn = (Ns_ + 63) / 64;
    pm.t_gu_wave = 2.0 * 256 * 256 * K_ / pair_rate;
    pm.t_dn_wave = 2.0 * 256 * 256 * Ns_ / pair_rate;
    pm.h2d_tile = (double)tile * K_ * 2 / 50e9;
    pm.d2h_tile = (double)tile * K_ * 2 / 45e9;
    std::vector<std::vector<int>> fam_g, fam_d;
    const int firsts[] = {1, 2, 3, 4};
    const double ratios[] = {1.0, 1.5, 2.0};
    const int caps[] = {4, 6, 8, 12, 16};
    for (int f : firsts) for (double q : ratios) for (int c : caps) {
        if (tiles > 256 && c < 8) continue;  // very large batches: keep the lists short
        std::vector<int> v = growing(tiles, f, q, c);
        fam_g.push_back(v);
        std::reverse(v.begin(), v.end());
        fam_d.push_back(v);
    }
    for (double frac : {0.5, 0.55, 0.6}) {  // halving sequence: most rows first, the rest in ever shorter chunks
        std::vector<int> v;
        int left = tiles;
        while (left > 0) {
            int c = std::max(1, std::min(left, (int)(left * frac + 0.999)));
            if (tiles > 256 && left * 2 < tiles && c < 8) c = std::min(left, 8);
            v.push_back(c);
            left -= c;
        }
        fam_d.push_back(v);
    }
    double best = 1e30;
    for (const auto& a : fam_g) for (const auto& b : fam_d) {
        const double t = pm.run(a, b);
        if (t < best) { best = t; g = a; d = b; }
    }
    finish(g); finish(d);
    if (cache) { cache->plan_M = M; cache->plan_gu = g; cache->plan_dn = d; }
    gu->swap(g); dn->swap(d);
}

int b200fc_mlp_host_plan(int M, int K, int N, int* gate_up_rows, int* down_rows, int capacity, int* n_gate_up, int* n_down) {
    if (M <= 0 || K <= 0 || N <= 0 || !gate_up_rows || !down_rows || !n_gate_up || !n_down || capacity <= 0) {
        set_error("mlp_host_plan: bad argument");
        return B200FC_ERR_INVALID;
    }
    std::vector<int> g, d;
    host_plan(nullptr, K, N, M, &g, &d);
    *n_gate_up = (int)g.size(); *n_down = (int)d.size();
    if ((int)g.size() > capacity || (int)d.size() > capacity) { set_error("mlp_host_plan: capacity too small"); return B200FC_ERR_INVALID; }
    for (size_t i = 0; i < g.size(); i++) gate_up_rows[i] = g[i];
    for (size_t i = 0; i < d.size(); i++) down_rows[i] = d[i];
    return B200FC_OK;
}

int b200fc_mlp_run_host(b200fc_mlp_t* h, const void* x, int64_t ldx, int M, void* out, int64_t ldo, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!h || !x || !out || M <= 0) { set_error("mlp_run_host: null pointer or M <= 0"); return B200FC_ERR_INVALID; }
    Mlp& m = h->m;
    if (m.tp_size != 1) { set_error("mlp_run_host: tensor-parallel shard"); return B200FC_ERR_INVALID; }
    const size_t row = (size_t)m.K * 2;
    int rc = grow(&m.stage_x, &m.stage_x_bytes, row * M, s);
    if (!rc) rc = grow(&m.stage_o, &m.stage_o_bytes, row * M, s);
    if (rc) return rc;
    static int pipe_min = -1;
    if (pipe_min < 0) { const char* e = getenv("B200FC_HOST_PIPE_MIN"); pipe_min = e ? atoi(e) : 512; }
    if (M < pipe_min) {
        B200FC_CUDA(cudaMemcpy2DAsync(m.stage_x, row, x, (size_t)ldx, row, (size_t)M, cudaMemcpyHostToDevice, s));
        rc = mlp_run_device(m, m.stage_x, (int64_t)row, M, m.stage_o, B200FC_BF16, (int64_t)row, s);
        if (rc) return rc;
        B200FC_CUDA(cudaMemcpy2DAsync(out, (size_t)ldo, m.stage_o, row, row, (size_t)M, cudaMemcpyDeviceToHost, s));
        return check_kernel_status(s);
    }
    // Large batches: rows are independent, so the batch flows through three streams — host-to-device copy,
    // compute, device-to-host copy — and the PCIe transfers overlap the tensor-core work (the copy engines are full
    // duplex).  The gate/up projection and the down projection are cut into row chunks independently of one
    // another (host_plan): short chunks at the head of the first and at the tail of the second keep the exposed
    // copies small, long chunks in between keep the GEMM waves full.
    std::vector<int> gu_rows, dn_rows;
    host_plan(&m, m.K, m.Ns, M, &gu_rows, &dn_rows);
    if (!m.pipe_streams[0]) {
        for (int i = 0; i < 3; i++) B200FC_CUDA(cudaStreamCreateWithFlags(&m.pipe_streams[i], cudaStreamNonBlocking));
        B200FC_CUDA(cudaEventCreateWithFlags(&m.ev_fork, cudaEventDisableTiming));
        B200FC_CUDA(cudaEventCreateWithFlags(&m.ev_join, cudaEventDisableTiming));
    }
    while (m.ev_in.size() < gu_rows.size() || m.ev_out.size() < dn_rows.size()) {
        cudaEvent_t a, b;
        B200FC_CUDA(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
        B200FC_CUDA(cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
        m.ev_in.push_back(a); m.ev_out.push_back(b);
    }
    rc = grow(&m.act, &m.act_bytes, (size_t)M * m.Ns * 2, s);
    if (rc) return rc;
    m.act_rows = M;
    cudaStream_t s_in = m.pipe_streams[0], s_cmp = m.pipe_streams[1], s_out = m.pipe_streams[2];
    B200FC_CUDA(cudaEventRecord(m.ev_fork, s));
    for (int i = 0; i < 3; i++) B200FC_CUDA(cudaStreamWaitEvent(m.pipe_streams[i], m.ev_fork, 0));
    size_t gi = 0;
    int gu_done = 0, d0 = 0;  // rows whose gate/up launch has been issued; first row of the next down chunk
    for (size_t j = 0; j < dn_rows.size(); j++) {
        const int d1 = d0 + dn_rows[j];
        while (gu_done < d1) {  // the activation rows this down chunk reads
            const int rows = gu_rows[gi];
            char* xs = (char*)m.stage_x + (size_t)gu_done * row;
            B200FC_CUDA(cudaMemcpy2DAsync(xs, row, (const char*)x + (size_t)gu_done * ldx, (size_t)ldx, row,
                                          (size_t)rows, cudaMemcpyHostToDevice, s_in));
            B200FC_CUDA(cudaEventRecord(m.ev_in[gi], s_in));
            B200FC_CUDA(cudaStreamWaitEvent(s_cmp, m.ev_in[gi], 0));
            b200fc_epilogue_t e1 = {};
            e1.steps = B200FC_STEP_SILU_MUL; e1.out_dtype = B200FC_BF16;
            e1.C = (char*)m.act + (size_t)gu_done * m.Ns * 2; e1.ldc_bytes = (int64_t)m.Ns * 2;
            rc = matmul_device(m.gate_up, nullptr, xs, B200FC_BF16, rows, m.K, (int64_t)row, 0, 2 * m.Ns, &e1, s_cmp);
            if (rc) return rc;
            gu_done += rows; gi++;
        }
        char* os = (char*)m.stage_o + (size_t)d0 * row;
        b200fc_epilogue_t e2 = {};
        e2.steps = 0; e2.out_dtype = B200FC_BF16; e2.C = os; e2.ldc_bytes = (int64_t)row;
        rc = matmul_device(m.down, nullptr, (char*)m.act + (size_t)d0 * m.Ns * 2, B200FC_BF16, d1 - d0, m.Ns,
                           (int64_t)m.Ns * 2, 0, m.K, &e2, s_cmp);
        if (rc) return rc;
        B200FC_CUDA(cudaEventRecord(m.ev_out[j], s_cmp));
        B200FC_CUDA(cudaStreamWaitEvent(s_out, m.ev_out[j], 0));
        B200FC_CUDA(cudaMemcpy2DAsync((char*)out + (size_t)d0 * ldo, (size_t)ldo, os, row, row, (size_t)(d1 - d0),
                                      cudaMemcpyDeviceToHost, s_out));
        d0 = d1;
    }
    B200FC_CUDA(cudaEventRecord(m.ev_join, s_out));
    B200FC_CUDA(cudaStreamWaitEvent(s, m.ev_join, 0));
    return check_kernel_status(s);
}

int b200fc_rmsnorm(const void* x, int64_t ldx, int M, int K, const void* weight, float eps, void* out, int64_t ldo,
                   void* stream) {
    if (!x || !out || M < 0 || K <= 0) { set_error("rmsnorm: null pointer or bad shape"); return B200FC_ERR_INVALID; }
    if (ldx < (int64_t)K * 2 || ldo < (int64_t)K * 2) { set_error("rmsnorm: leading dimension smaller than a row"); return B200FC_ERR_INVALID; }
    return launch_rmsnorm(x, ldx, M, K, weight, eps, out, ldo, (cudaStream_t)stream);
}

int b200fc_mlp_run_block(b200fc_mlp_t* h, const void* x, int64_t ldx, int M, float eps, const void* norm_weight,
                         int add_residual, void* out, int64_t ldo, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!h || !x || !out) { set_error("mlp_run_block: null pointer"); return B200FC_ERR_INVALID; }
    Mlp& m = h->m;
    if (m.tp_size != 1) { set_error("mlp_run_block: tensor-parallel shard"); return B200FC_ERR_INVALID; }
    if (M < 0) { set_error("mlp_run_block: M < 0"); return B200FC_ERR_INVALID; }
    if (M == 0) return B200FC_OK;
    // normalised activations: per-stream scratch (kernels on one stream are ordered)
    void* xn = nullptr;
    const int64_t ldn = (int64_t)m.K * 2;
    int rc = get_stream_scratch((size_t)M * ldn, s, 4, &xn);
    if (!rc) rc = launch_rmsnorm(x, ldx, M, m.K, norm_weight, eps, xn, ldn, s);
    if (!rc && M <= 16) {
        rc = grow(&m.act, &m.act_bytes, (size_t)M * m.Ns * 2, s);
        if (!rc) rc = mlp_decode_fused_device(m, xn, ldn, M, m.act, out, B200FC_BF16, ldo, s, nullptr, add_residual ? x : nullptr, ldx);
        if (rc != B200FC_ERR_UNSUPPORTED) {
            if (!rc) m.act_rows = M;
            return rc;
        }
        rc = B200FC_OK;
    }
    if (!rc) rc = mlp_gate_up_device(m, xn, ldn, M, s);
    if (rc) return rc;
    b200fc_epilogue_t e2 = {};
    e2.steps = 0; e2.out_dtype = B200FC_BF16; e2.C = out; e2.ldc_bytes = ldo;
    return matmul_device(m.down, nullptr, m.act, B200FC_BF16, M, m.Ns, (int64_t)m.Ns * 2, 0, m.K, &e2, s, nullptr,
                         add_residual ? x : nullptr, ldx);
}

const void* b200fc_mlp_act(const b200fc_mlp_t* h) { return h ? h->m.act : nullptr; }

int b200fc_decode_attention(const b200fc_attention_t* a, void* stream) {
    if (!a) { set_error("decode_attention: null descriptor"); return B200FC_ERR_INVALID; }
    return launch_decode_attention(*a, (cudaStream_t)stream);
}

int b200fc_device_malloc(void** ptr, int64_t bytes) {
    if (!ptr || bytes < 0) { set_error("device_malloc: bad argument"); return B200FC_ERR_INVALID; }
    B200FC_CUDA(cudaMalloc(ptr, (size_t)(bytes > 0 ? bytes : 1)));
    return B200FC_OK;
}
int b200fc_device_free(void* ptr) {
    B200FC_CUDA(cudaFree(ptr));
    return B200FC_OK;
}
int b200fc_memcpy(void* dst, const void* src, int64_t bytes, void* stream) {
    if (bytes < 0 || (bytes > 0 && (!dst || !src))) { set_error("memcpy: bad argument"); return B200FC_ERR_INVALID; }
    B200FC_CUDA(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, (cudaStream_t)stream));
    B200FC_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return B200FC_OK;
}

int b200fc_add_round_bf16(const float* a, const float* b, void* out, int64_t n, void* stream) {
    if (!a || !out || n < 0) { set_error("add_round_bf16: bad argument"); return B200FC_ERR_INVALID; }
    return launch_add_round_bf16(a, b, out, n, (cudaStream_t)stream);
}

int b200fc_flush_l2(void* stream) {
    static std::map<int, void*> bufs;               // one buffer per device, under g_mu
    static const size_t bytes = (size_t)256 << 20;  // twice the 126 MB L2
    int dev = 0;
    B200FC_CUDA(cudaGetDevice(&dev));
    void* buf = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = bufs.find(dev);
        if (it == bufs.end()) {
            B200FC_CUDA(cudaMalloc(&buf, bytes));
            bufs[dev] = buf;
        } else {
            buf = it->second;
        }
    }
    return launch_fill(buf, bytes, (cudaStream_t)stream);
}

}  // extern "C"
