// Shared declarations of the b200fc library: packed-weight object, kernel launch entry points, post-op math.
#pragma once
#include <atomic>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <vector>
#include "../../include/b200fc.h"

namespace b200fc {

// ---------------------------------------------------------------------------------------------------------------
// Packed weights.  One layout serves every kernel: a row-major [N_pad, K_pad] matrix with K contiguous
// ("K-major"), zero padded.  A 2-D TMA box of it with 128-byte swizzle lands in shared memory in the canonical
// tcgen05 K-major operand layout; the decode kernels stream its rows with 16-byte loads.
//   K_pad: multiple of 128 bytes of elements (64 bf16 / 128 int8 / 256 four-bit)     N_pad: multiple of 256 rows
// 4-bit weights (dtype B200FC_S4) keep the row-major byte matrix, two values per byte, with K permuted inside every
// 128-byte piece of a row for the decode kernel (see quant4_kernel in pack.cu), and carry group scales.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kRowPad = 256;
constexpr int kKPadBytes = 128;

struct Weight {
    int K = 0, N = 0;
    int K_pad = 0, N_pad = 0;
    int dtype = B200FC_BF16;        // stored element type: BF16, S8, U8
    bool compressed = false;        // int8 weights used with bf16 activations; stored offset-binary (value + 128)
    float deq_scale = 1.0f;         // per-tensor dequant scale of compressed weights
    void* data = nullptr;           // [N_pad, K_pad]
    float* scale_per_oc = nullptr;  // optional [N_pad] per-output-channel dequant scales
    float* scale_grp = nullptr;     // 4-bit weights: [N_pad / 128][K_pad / 256][2][128] dequant scales, i.e. for every
                                    // 128-row x 128-byte piece of the packed matrix the 2 x 128 scales it needs, contiguous
    // lazily created scratch / staging owned by the object
    void* stage_A = nullptr; size_t stage_A_bytes = 0;
    void* stage_C = nullptr; size_t stage_C_bytes = 0;
    float* stage_vec = nullptr; size_t stage_vec_floats = 0;
    int64_t ld_bytes() const { return dtype == B200FC_S4 ? (int64_t)K_pad / 2 : (int64_t)K_pad * (dtype == B200FC_BF16 ? 2 : 1); }
    size_t data_bytes() const { return (size_t)N_pad * (size_t)ld_bytes(); }
    size_t scale_grp_floats() const { return dtype == B200FC_S4 ? (size_t)N_pad * (size_t)(K_pad / 128) : 0; }
};

// Post-op description handed to kernels (device pointers).
struct Epilogue {
    int steps;
    int out_dtype;
    void* C;
    long long ldc;  // bytes
    const float* bias;
    float deq_scale;
    const float* deq_per_oc;
    float q_scale;
    const float* q_per_oc;
    int mc_reduce = 0;  // 1: C is an NVLink multicast address; the store is a multimem.red.add (in-switch all-reduce)
    // optional residual, added in fp32 right before the output is rounded: C[m, n] = round(post-ops(...) + residual[m, n])
    const void* residual = nullptr;   // [M, N] bf16
    long long ld_res = 0;             // bytes
};

// Fused Llama MLP object (b200fc_mlp_t)
struct Mlp {
    int K = 0, N = 0, Ns = 0;  // hidden, intermediate, this rank's share of the intermediate dimension
    int tp_rank = 0, tp_size = 1;
    Weight gate_up, down;
    void* act = nullptr; size_t act_bytes = 0;      // [M, Ns] bf16
    int act_rows = 0;                               // rows of the last gate_up
    void* stage_x = nullptr; size_t stage_x_bytes = 0;
    void* stage_o = nullptr; size_t stage_o_bytes = 0;
    // host-buffer entry point, large batches: copy-in / compute / copy-out streams and their events
    cudaStream_t pipe_streams[3] = {nullptr, nullptr, nullptr};
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    std::vector<cudaEvent_t> ev_in, ev_out;
    int plan_M = 0;                                 // row chunks of that pipeline, as planned for plan_M rows
    std::vector<int> plan_gu, plan_dn;
};

// cudaFuncSetAttribute applies to the current device only.  Runs `set_attr` (returns a status code) the first time
// the calling launcher is used on a device and remembers the device in `mask` (one bit per device ordinal); two
// threads racing on the first use both set the attribute, which is harmless.
template <typename F>
inline int once_per_device(std::atomic<unsigned long long>& mask, F&& set_attr) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
    const unsigned long long bit = 1ull << (dev & 63);
    if (mask.load(std::memory_order_acquire) & bit) return 0;
    const int rc = set_attr();
    if (!rc) mask.fetch_or(bit, std::memory_order_release);
    return rc;
}

// SM budget of the persistent GEMM grids (0 = all SMs); set through b200fc_set_sm_limit
int sm_limit();

// error plumbing (api.cu)
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
void count_launch(int n = 1);
int* kernel_status_word();  // device int, 0 = OK; kernels store a non-zero code when a bounded wait runs out
int check_kernel_status(cudaStream_t s);  // synchronises and reads it
// growing device scratch owned by (device, stream, slot): work on one stream is ordered, so kernels launched on it
// may share it; slot 0 = re-strided activations, slot 1 = split-K partial tiles of the GEMM, 3 = widened weight
// rows, 4 = normalised activations of the MLP block, 5 = sub-states of the decode attention, 6 = pre-converted activations
// of the decode kernel
int get_stream_scratch(size_t bytes, cudaStream_t s, int slot, void** out);
// the decode kernel's scratch for stream s (gemv_scratch_bytes(), counters zero); never re-allocated once handed out
int get_gemv_scratch(cudaStream_t s, void** out);
// time limit of every bounded device-side wait (b200fc_set_wait_limit_ns; 2 s unless changed)
unsigned long long wait_limit_ns();

#define B200FC_CUDA(call)                                                   \
    do {                                                                    \
        cudaError_t e__ = (call);                                           \
        if (e__ != cudaSuccess) return ::b200fc::cuda_fail(e__, #call);     \
    } while (0)

// api.cu: gate/up + down of a decode-shaped MLP (1 <= M <= 16) in one launch; B200FC_ERR_UNSUPPORTED without a message =
// not possible here, launch the two projections separately
int mlp_decode_fused_device(const Mlp& m, const void* x, int64_t ldx, int M, void* act, void* out, int out_dtype,
                            int64_t ldo, cudaStream_t s, void* gemv_scratch, const void* residual, int64_t ld_res);
// api.cu: validated dispatch of one Matmul call on device pointers (w_mut is unused and kept for call-site symmetry)
// gemv_scratch: counters + partial-sum slots for the decode kernel (gemv_scratch_bytes(), counters zero), or null to
// use the stream's own
// residual: optional [M, N] bf16 matrix added to the result before the output rounding (not with SILU_MUL)
int matmul_device(const Weight& w, Weight* w_mut, const void* A, int dtypeA, int M, int K, int64_t lda, int n0, int n1,
                  const b200fc_epilogue_t* ep, cudaStream_t s, void* gemv_scratch = nullptr,
                  const void* residual = nullptr, int64_t ld_res = 0);

// ---- launchers -------------------------------------------------------------------------------------------------
// pack.cu
int launch_pack(const void* B_dev, int dtypeB, int K, int N, int64_t ldb, int transposeB, Weight& w, bool offset_binary,
                cudaStream_t s);
int launch_flip_copy2d(const void* src, int64_t lds, void* dst, int64_t ldd, int rows, int cols, cudaStream_t s);
int launch_pack_gate_up(const void* gate, const void* up, int64_t ld_bytes, int K, int rows, Weight& w, cudaStream_t s);
int launch_quant_pack(const void* B_dev, int K, int N, int64_t ldb, int transposeB, Weight& w, float* absmax_dev,
                      cudaStream_t s);
int launch_absmax(const void* B_dev, int rows, int cols, int64_t ldb, float* absmax_dev, cudaStream_t s);
int launch_dequant_bf16(const Weight& w, int row0, int rows, void* dst_bf16, int dst_K_pad, cudaStream_t s);
// 4-bit weights: bf16 [N_pad, K_pad] K-major (zero padded) -> w.data / w.scale_grp; and back to one int8 per value
int launch_quant4(const void* wide_bf16, Weight& w, cudaStream_t s);
int launch_unpack4(const Weight& w, void* dst_s8, int64_t ldd, cudaStream_t s);
int launch_copy2d(const void* src, int64_t lds, void* dst, int64_t ldd, int rows, int row_bytes, int dst_row_bytes,
                  cudaStream_t s);
int launch_add_round_bf16(const float* a, const float* b, void* out, int64_t n, cudaStream_t s);
int launch_fill(void* p, size_t bytes, cudaStream_t s);
int launch_rmsnorm(const void* x, int64_t ldx, int M, int K, const void* weight, float eps, void* out, int64_t ldo,
                   cudaStream_t s);
// gemv_tma.cu: M <= 16, bf16 activations, bf16 or int8 weights streamed by TMA through a shared-memory ring.
// `scratch`: gemv_scratch_bytes() of device memory whose first kGemvMaxCtas words are zero (the kernel leaves them
// zero), shared by the launches of one stream; null = the stream's own (allocated on first use).
constexpr int kGemvMaxCtas = 320;
size_t gemv_scratch_bytes();
void set_decode_ctas_per_sm(int n);
int launch_gemv_tma(const Weight& w, const void* A, int M, int K, int64_t lda, int n0, int n1, const Epilogue& ep,
                    cudaStream_t s, void* scratch);
// gemv_tma.cu: gate/up + down of a decode-shaped MLP (bf16 weights, M <= 16) in one launch; B200FC_ERR_UNSUPPORTED
// without a message = not possible for this shape / device, launch the two matrices one after the other
int launch_mlp_decode_fused(const Weight& gate_up, const Weight& down, const void* x, int64_t ldx, int M, int K, int ns,
                            void* act, const Epilogue& ep_down, cudaStream_t s, void* scratch);
// gemm_tc.cu: tcgen05 GEMM, bf16 x bf16 -> fp32 or 8-bit x 8-bit -> int32
int launch_gemm_tc(const void* W_data, int w_dtype, int W_K_pad, int W_N_pad, const void* A, int dtypeA, int M, int K,
                   int64_t lda, int n0, int n1, const Epilogue& ep, cudaStream_t s);
// gemm_tc.cu: bf16 GEMM whose output is all-reduced over a tensor-parallel group inside the kernel
struct AllReduceDesc {
    int world, rank;
    void* partial_local;      // this rank's replica of the symmetric partial buffer [M, N] bf16
    const void* partial_mc;   // multicast address of all replicas of it
    void* out_mc;             // multicast address of all replicas of the output buffer [M, N] bf16
    int64_t ld_bytes;         // row pitch of both buffers
    unsigned* flags[8];       // per rank: arrival counters, one per tile, zero before the call
    int max_tiles;            // length of the counter arrays
    int comm_sms;             // SMs given to the reducing role
};
int launch_gemm_tc_allreduce(const void* W_data, int W_K_pad, int W_N_pad, const void* A, int M, int K, int64_t lda,
                             int N, const AllReduceDesc& ar, cudaStream_t s);
// attention.cu
int launch_decode_attention(const b200fc_attention_t& a, cudaStream_t s);
// matvec.cu
int launch_matvec(const void* A, int dtype, int M, int K, int64_t lda, const void* b, void* c, cudaStream_t s);

// ---------------------------------------------------------------------------------------------------------------
// Post-op math shared by all kernels (device).
// ---------------------------------------------------------------------------------------------------------------
#ifdef __CUDACC__

// erf-GeLU through the minimax polynomial in x^2 that the reference evaluates (gelu_erf_minmax_approx,
// include/kernels_amx.hpp:242-289): x < -5 -> 0, |x| > 5 -> x, |x| <= 2^-24 -> x/2, else x/2 * (1 + x * P(x^2)).
__device__ __forceinline__ float gelu_erf_poly(float x) {
    const float x2 = x * x, ax = fabsf(x), xh = 0.5f * x;
    float p = __uint_as_float(0x1f1c83fdu);
    p = fmaf(p, x2, __uint_as_float(0xa3198977u));
    p = fmaf(p, x2, __uint_as_float(0x268a7927u));
    p = fmaf(p, x2, __uint_as_float(0xa998c963u));
    p = fmaf(p, x2, __uint_as_float(0x2c67ddb2u));
    p = fmaf(p, x2, __uint_as_float(0xaf013b2cu));
    p = fmaf(p, x2, __uint_as_float(0x315d4a4fu));
    p = fmaf(p, x2, __uint_as_float(0xb3969b11u));
    p = fmaf(p, x2, __uint_as_float(0x35a776e9u));
    p = fmaf(p, x2, __uint_as_float(0xb79b0914u));
    p = fmaf(p, x2, __uint_as_float(0x3970b255u));
    p = fmaf(p, x2, __uint_as_float(0xbb1b7399u));
    p = fmaf(p, x2, __uint_as_float(0x3ca3621fu));
    p = fmaf(p, x2, __uint_as_float(0xbe082bc7u));
    p = fmaf(p, x2, __uint_as_float(0x3f4c4228u));
    p = fmaf(p, x, 1.0f) * xh;
    if (x < -5.0f) x = 0.0f;
    if (!(ax <= 5.0f)) p = x;
    if (ax <= __uint_as_float(0x33800000u)) p = xh;
    return p;
}

// SiLU of the fused MLP (silu_ps_avx512, tests/amx-mlp.cpp:445-451): x / (1 + exp(-x)).  The reference pairs a
// degree-5 exp polynomial with a 14-bit reciprocal; here expf and a true division (differences <= ~2^-13 relative,
// below the bf16 rounding that follows).
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// fp32 -> int8 like VCVTPS2DQ + VPMOVSDB (include/kernels_amx.hpp:657-664): round to nearest even, saturate; NaN -> -128.
__device__ __forceinline__ int f32_to_s8(float v) {
    if (v != v) return -128;
    int r;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}

__device__ __forceinline__ unsigned short f32_to_bf16_bits(float v) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}

// DEQUANT -> BIAS -> GELU -> QUANT on one fp32 value of output column n.
__device__ __forceinline__ float postop_scalar(float v, int n, const Epilogue& ep) {
    if (ep.steps & B200FC_STEP_DEQUANT) v *= ep.deq_per_oc ? ep.deq_scale * __ldg(ep.deq_per_oc + n) : ep.deq_scale;
    if (ep.steps & B200FC_STEP_BIAS) v += __ldg(ep.bias + n);
    if (ep.steps & B200FC_STEP_GELU) v = gelu_erf_poly(v);
    if (ep.steps & B200FC_STEP_QUANT) v *= ep.q_per_oc ? __ldg(ep.q_per_oc + n) : ep.q_scale;
    return v;
}

__device__ __forceinline__ float residual_at(const Epilogue& ep, int m, int n) {
    const unsigned short b = ((const unsigned short*)((const char*)ep.residual + (long long)m * ep.ld_res))[n];
    return __uint_as_float((unsigned)b << 16);
}

__device__ __forceinline__ void store_scalar(float v, int m, int n, const Epilogue& ep) {
    if (ep.residual) v += residual_at(ep, m, n);
    char* row = (char*)ep.C + (long long)m * ep.ldc;
    if (ep.out_dtype == B200FC_F32) ((float*)row)[n] = v;
    else if (ep.out_dtype == B200FC_BF16) ((unsigned short*)row)[n] = f32_to_bf16_bits(v);
    else ((signed char*)row)[n] = (signed char)f32_to_s8(v);
}

#endif  // __CUDACC__

}  // namespace b200fc

// the opaque handle types of the C ABI
struct b200fc_weight { b200fc::Weight w; };
struct b200fc_mlp { b200fc::Mlp m; };
