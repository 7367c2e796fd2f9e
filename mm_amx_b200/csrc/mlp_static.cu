// Decode-shaped fused MLP that never allocates.
//
// Some callers are not allowed to enter the CUDA allocator once they are running: a serving loop whose memory plan
// was fixed at start-up and that hands every remaining byte of HBM to a KV cache, a callback running while another
// thread holds an allocator lock, a host runtime that forbids any cudaMalloc / cudaFree after initialisation because
// those calls synchronise the device.  b200fc_mlp_run keeps its gate/up activation in a buffer that it grows with
// cudaMalloc on demand, so those callers cannot use it.  The entry point below does the same computation for
// decode-shaped batches with the activation held in a fixed device array that is part of this library's image.
//
// The decode kernel itself also needs a little global scratch (partial sums of weight-row blocks that two SMs share,
// and their arrival counters), which the ordinary entry points take from a per-stream allocation; here it is a second
// fixed device array.
//
// It has no counterpart in the reference (whose activation buffer grows inside MLP::run).
#include <map>
#include <mutex>
#include "common.cuh"

namespace {

// The scratch: one activation matrix [M, N / tp] in bf16.  Every GPU that loads this library holds these bytes from
// load until the process exits.
constexpr size_t kStaticActBytes = (size_t)1 << 20;  // 1 MiB: M * (N / tp) <= 524288 elements, e.g. 16 rows x 28672
static __device__ __align__(256) unsigned char g_static_act[kStaticActBytes];

// The decode kernel's counters (first, zero from load and left zero by every launch) and partial-sum slots.
constexpr size_t kStaticGemvBytes = (size_t)b200fc::kGemvMaxCtas * (2 * 16 * 128 * sizeof(float) + sizeof(unsigned));
static __device__ __align__(256) unsigned char g_static_gemv[kStaticGemvBytes];

struct StaticAddr { void* act; void* gemv; };
std::mutex g_mu;
std::map<int, StaticAddr> g_addr;  // device ordinal -> device addresses of the two arrays on that device

// In host code the name g_static_act is only a handle for the symbol, not a device address; the address has to be
// asked for, once per device, with that device current.
int static_addresses(StaticAddr* out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return b200fc::cuda_fail(e, "cudaGetDevice");
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_addr.find(dev);
    if (it == g_addr.end()) {
        if (b200fc::gemv_scratch_bytes() > kStaticGemvBytes) { b200fc::set_error("mlp_run_decode_static: internal scratch size mismatch"); return B200FC_ERR_INVALID; }
        StaticAddr a = {nullptr, nullptr};
        e = cudaGetSymbolAddress((void**)&a.act, g_static_act);
        if (e != cudaSuccess) return b200fc::cuda_fail(e, "cudaGetSymbolAddress(g_static_act)");
        e = cudaGetSymbolAddress((void**)&a.gemv, g_static_gemv);
        if (e != cudaSuccess) return b200fc::cuda_fail(e, "cudaGetSymbolAddress(g_static_gemv)");
        if (!a.act || !a.gemv) { b200fc::set_error("mlp_run_decode_static: null symbol address"); return B200FC_ERR_CUDA; }
        it = g_addr.emplace(dev, a).first;
    }
    *out = it->second;
    return B200FC_OK;
}

}  // namespace

extern "C" {

int64_t b200fc_mlp_decode_static_capacity(void) { return (int64_t)kStaticActBytes; }
int64_t b200fc_mlp_decode_static_footprint(void) { return (int64_t)(kStaticActBytes + kStaticGemvBytes); }

int b200fc_mlp_run_decode_static(b200fc_mlp_t* h, const void* x, int64_t ldx, int M, void* out, int out_dtype,
                                 int64_t ldo, void* stream) {
    using namespace b200fc;
    cudaStream_t s = (cudaStream_t)stream;
    if (!h || !x || !out) { set_error("mlp_run_decode_static: null pointer"); return B200FC_ERR_INVALID; }
    if (out_dtype != B200FC_BF16 && out_dtype != B200FC_F32) { set_error("mlp_run_decode_static: out_dtype must be bf16 or f32"); return B200FC_ERR_INVALID; }
    Mlp& m = h->m;
    if (M < 1 || M > 16) {
        set_error("mlp_run_decode_static: M = %d outside [1, 16] (decode-shaped batches only)", M);
        return B200FC_ERR_INVALID;
    }
    const size_t need = (size_t)M * m.Ns * 2;
    if (need > kStaticActBytes) {
        set_error("mlp_run_decode_static: activation of %d x %d bf16 = %zu bytes exceeds the fixed %zu-byte scratch",
                  M, m.Ns, need, kStaticActBytes);
        return B200FC_ERR_INVALID;
    }
    StaticAddr addr;
    int rc = static_addresses(&addr);
    if (rc) return rc;
    void* act = addr.act;
    // gate/up projection + SiLU*up writes all M x Ns activation elements before the down projection reads them, and
    // the down projection reads nothing beyond them, so nothing in the activation array has to be cleared between
    // calls.  The decode kernel writes every partial-sum slot before it reads it and returns its counters to zero.
    rc = mlp_decode_fused_device(m, x, ldx, M, act, out, out_dtype, ldo, s, addr.gemv, nullptr, 0);   // one launch if possible
    if (rc != B200FC_ERR_UNSUPPORTED) return rc;
    b200fc_epilogue_t e1 = {};
    e1.steps = B200FC_STEP_SILU_MUL; e1.out_dtype = B200FC_BF16; e1.C = act; e1.ldc_bytes = (int64_t)m.Ns * 2;
    rc = matmul_device(m.gate_up, nullptr, x, B200FC_BF16, M, m.K, ldx, 0, 2 * m.Ns, &e1, s, addr.gemv);
    if (rc) return rc;
    b200fc_epilogue_t e2 = {};
    e2.steps = 0; e2.out_dtype = out_dtype; e2.C = out; e2.ldc_bytes = ldo;
    return matmul_device(m.down, nullptr, act, B200FC_BF16, M, m.Ns, (int64_t)m.Ns * 2, 0, m.K, &e2, s, addr.gemv);
}

}  // extern "C"
