// TEST INFRASTRUCTURE — the parity oracle.  Never linked into, imported by, or called from the shipped library.
//
// Plain C++ (no intrinsics, no CUDA) restatement of the arithmetic of the fully-connected hot path of
// usstq/mm_amx, so it runs on any host.  Every function cites the reference file:line it follows.  It is pinned
// against the reference's own AMX code (oracle/ref_harness.cpp) by tests/golden/make_golden.py and by
// tests/test_oracle_vs_ref.py on hosts that have AMX.
//
// Conventions: bf16 values travel as uint16_t bit patterns; all strides are in BYTES (tensor2D::stride,
// include/tensor2D.hpp:34); matrices are row-major.  Build: make -C oracle  (-ffp-contract=off: fused operations are
// written out with fmaf where the reference uses an FMA instruction).
#include <cstdint>
#include <cstring>
#include <cmath>
#include <vector>
#include <algorithm>
#include <omp.h>

namespace {

inline float bf2f(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }
inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

// fp32 -> bf16 as the VCVTNE2PS2BF16 instruction used by the post-op store (include/kernels_amx.hpp:653-656) and
// ov::bfloat16::round_to_nearest_even (include/bf16.hpp:91-102): round to nearest even on the upper 16 bits;
// zero/denormal inputs give signed zero, NaN is quieted.
inline uint16_t f2bf(float f) {
    uint32_t u = f2u(f);
    uint32_t exp = (u >> 23) & 0xff, man = u & 0x7fffff;
    if (exp == 0) return (uint16_t)((u >> 16) & 0x8000);
    if (exp == 0xff) return (uint16_t)((u >> 16) | (man ? 0x40 : 0));
    return (uint16_t)((u + 0x7fff + ((u >> 16) & 1)) >> 16);
}

// erf-based GeLU, minimax polynomial in x^2 (include/kernels_amx.hpp:242-289): zones x < -5 -> 0, |x| > 5 -> x,
// |x| <= 2^-24 -> x/2, else x/2 * (1 + x*P(x^2)), P evaluated by Horner with FMAs.
const uint32_t kGeluPoly[15] = {0x1f1c83fd, 0xa3198977, 0x268a7927, 0xa998c963, 0x2c67ddb2, 0xaf013b2c, 0x315d4a4f,
                                0xb3969b11, 0x35a776e9, 0xb79b0914, 0x3970b255, 0xbb1b7399, 0x3ca3621f, 0xbe082bc7,
                                0x3f4c4228};
inline float gelu(float x) {
    float x2 = x * x, ax = std::fabs(x), xh = x * 0.5f;
    float p = u2f(kGeluPoly[0]);
    for (int i = 1; i < 15; i++) p = fmaf(p, x2, u2f(kGeluPoly[i]));
    p = fmaf(p, x, 1.0f);
    p = p * xh;
    if (x < -5.0f) x = 0.0f;            // zone 1 (NaN keeps x)
    if (!(ax <= 5.0f)) p = x;           // zone 5 and zone 1 (and NaN)
    if (ax <= u2f(0x33800000)) p = xh;  // zone 3
    return p;
}

// exp(x) of tests/amx-mlp.cpp:383-443: clamp to [ln FLT_MIN, ln FLT_MAX], n = floor(x*log2e + 0.5),
// r = x - n*ln2, degree-5 polynomial in r, scaled by 2 * 2^(n-1); inputs below ln FLT_MIN give 0.
inline float exp_poly(float x) {
    const float lo = u2f(0xc2aeac50), hi = u2f(0x42b17218);
    bool under = x < lo;
    x = std::max(std::min(x, hi), lo);
    float n = std::floor(x * u2f(0x3fb8aa3b) + 0.5f);
    float r = fmaf(-n, u2f(0x3f317218), x);
    int32_t e = (int32_t)std::nearbyintf(n - 1.0f);
    float scale = under ? 0.0f : u2f((uint32_t)(e + 127) << 23);
    float p = u2f(0x3c07cfce);
    p = fmaf(p, r, u2f(0x3d2b9d0d));
    p = fmaf(p, r, u2f(0x3e2aad40));
    p = fmaf(p, r, u2f(0x3efffee3));
    p = fmaf(p, r, u2f(0x3f7ffffb));
    p = fmaf(p, r, 1.0f);
    return p * scale * 2.0f;
}
// SiLU of tests/amx-mlp.cpp:445-451: x * rcp(1 + exp(-x)).  The reference uses the approximate reciprocal
// VRCP14PS (relative error <= 2^-14, table not restatable); this port divides exactly, so results may differ
// from the reference by up to 2^-14 relative before the bf16 rounding of the activation.
inline float silu(float x) { return x * (1.0f / (1.0f + exp_poly(0.0f - x))); }

// int8 store of the post-op (include/kernels_amx.hpp:657-664): VCVTPS2DQ under the default rounding mode (nearest
// even; NaN and out-of-range give INT_MIN) followed by signed saturation to 8 bits.
inline int8_t f2s8(float v) {
    int32_t i;
    if (!(v > -2147483648.0f && v < 2147483648.0f)) i = INT32_MIN;
    else i = (int32_t)std::nearbyintf(v);
    return (int8_t)std::max(-128, std::min(127, i));
}

enum Steps { DEQUANT = 1, BIAS = 2, GELU = 4, QUANT = 8 };  // PP::Steps, include/kernels_amx.hpp:540-550

}  // namespace

extern "C" {

int orc_threads() { return omp_get_max_threads(); }

void orc_f32_to_bf16(const float* x, uint16_t* y, int64_t n) { for (int64_t i = 0; i < n; i++) y[i] = f2bf(x[i]); }
void orc_gelu(const float* x, float* y, int64_t n) { for (int64_t i = 0; i < n; i++) y[i] = gelu(x[i]); }
void orc_silu(const float* x, float* y, int64_t n) { for (int64_t i = 0; i < n; i++) y[i] = silu(x[i]); }

// fp32 accumulators of A[M,K] (bf16) x B (bf16; [K,N], or [N,K] when transposeB) as TDPBF16PS produces them in
// Matmul::operator() (include/kernels_amx.hpp:1169-1314): k advances in 32-element tiles; inside a tile the 16
// bf16 pairs are consumed in order and within a pair the odd element's product is added after the even one's —
// every product is exact in fp32, every addition rounds to nearest even.  A K tail (K % 32) is the last,
// zero-padded tile (include/kernels_amx.hpp:1276-1289), i.e. the same order.
void orc_gemm_bf16(const uint16_t* A, int64_t lda, const uint16_t* B, int64_t ldb, int transposeB, int M, int K, int N,
                   float* acc, int64_t ld_acc_elems) {
    std::vector<float> Af((size_t)M * K), Bt((size_t)N * K);
    #pragma omp parallel for
    for (int m = 0; m < M; m++) {
        const uint16_t* a = (const uint16_t*)((const uint8_t*)A + m * lda);
        for (int k = 0; k < K; k++) Af[(size_t)m * K + k] = bf2f(a[k]);
    }
    if (transposeB) {
        #pragma omp parallel for
        for (int n = 0; n < N; n++) {
            const uint16_t* b = (const uint16_t*)((const uint8_t*)B + n * ldb);
            for (int k = 0; k < K; k++) Bt[(size_t)n * K + k] = bf2f(b[k]);
        }
    } else {
        #pragma omp parallel for
        for (int k = 0; k < K; k++) {
            const uint16_t* b = (const uint16_t*)((const uint8_t*)B + k * ldb);
            for (int n = 0; n < N; n++) Bt[(size_t)n * K + k] = bf2f(b[n]);
        }
    }
    const int NB = 8;
    #pragma omp parallel for collapse(2) schedule(static)
    for (int m = 0; m < M; m++) {
        for (int n0 = 0; n0 < N; n0 += NB) {
            int nb = std::min(NB, N - n0);
            float s[NB] = {0};
            const float* a = &Af[(size_t)m * K];
            for (int k = 0; k < K; k++) {
                float av = a[k];
                for (int j = 0; j < nb; j++) s[j] = s[j] + av * Bt[(size_t)(n0 + j) * K + k];
            }
            for (int j = 0; j < nb; j++) acc[(size_t)m * ld_acc_elems + n0 + j] = s[j];
        }
    }
}

// exact int32 accumulators of int8 x int8 (TDPBSSD and its unsigned variants, include/kernels_amx.hpp:1096-1101).
// a_unsigned / b_unsigned select the u8 interpretations.
void orc_gemm_i8(const void* A, int64_t lda, int a_unsigned, const void* B, int64_t ldb, int b_unsigned, int transposeB,
                 int M, int K, int N, int32_t* acc, int64_t ld_acc_elems) {
    std::vector<int16_t> Bt((size_t)N * K);
    #pragma omp parallel for
    for (int n = 0; n < N; n++)
        for (int k = 0; k < K; k++) {
            const uint8_t* p = (const uint8_t*)B + (transposeB ? (n * ldb + k) : (k * ldb + n));
            Bt[(size_t)n * K + k] = b_unsigned ? (int16_t)*p : (int16_t)*(const int8_t*)p;
        }
    #pragma omp parallel for collapse(2) schedule(static)
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++) {
            const uint8_t* a = (const uint8_t*)A + m * lda;
            const int16_t* b = &Bt[(size_t)n * K];
            int32_t s = 0;
            for (int k = 0; k < K; k++) {
                int32_t av = a_unsigned ? (int32_t)a[k] : (int32_t)(int8_t)a[k];
                s += av * (int32_t)b[k];
            }
            acc[(size_t)m * ld_acc_elems + n] = s;
        }
}

// PP::BiasGeluStore::operator() (include/kernels_amx.hpp:586-672) on a whole accumulator matrix.  Fixed order:
// [int32 -> fp32] -> DEQUANT (* deq_scale; deq_scale_per_oc[n] is this project's per-channel extension, applied as
// one multiply by deq_scale*deq_scale_per_oc[n]) -> BIAS -> GELU -> QUANT (* q_scale or q_scale_per_oc[n]) ->
// store as fp32 (out_dtype 0), bf16 (1) or int8 (2).
void orc_postops(const void* acc, int acc_is_int32, int64_t ld_acc_elems, int M, int N, int steps, float deq_scale,
                 const float* deq_scale_per_oc, const float* bias, float q_scale, const float* q_scale_per_oc,
                 int out_dtype, void* C, int64_t ldc) {
    #pragma omp parallel for
    for (int m = 0; m < M; m++) {
        uint8_t* row = (uint8_t*)C + m * ldc;
        for (int n = 0; n < N; n++) {
            float v = acc_is_int32 ? (float)((const int32_t*)acc)[(size_t)m * ld_acc_elems + n]
                                   : ((const float*)acc)[(size_t)m * ld_acc_elems + n];
            if (steps & DEQUANT) v = v * (deq_scale_per_oc ? deq_scale * deq_scale_per_oc[n] : deq_scale);
            if (steps & BIAS) v = v + bias[n];
            if (steps & GELU) v = gelu(v);
            if (steps & QUANT) v = v * (q_scale_per_oc ? q_scale_per_oc[n] : q_scale);
            if (out_dtype == 0) ((float*)row)[n] = v;
            else if (out_dtype == 1) ((uint16_t*)row)[n] = f2bf(v);
            else ((int8_t*)row)[n] = f2s8(v);
        }
    }
}

// Per-tensor symmetric int8 quantisation of bf16 weights as the compressed Matmul does on its first call
// (include/kernels_amx.hpp:1363-1377 with get_min_max :465-488 and bf16_to_i8_tensor :508-523):
// quant = 127/absmax, q = saturate_s8(round_nearest_even(w * quant)), dequant = absmax/127.
// Wq gets the same [rows, cols] shape as W (compact).
void orc_quantize_weight(const uint16_t* W, int64_t ldw, int rows, int cols, int8_t* Wq, float* quant, float* dequant) {
    float mx = 0.0f;
    for (int r = 0; r < rows; r++) {
        const uint16_t* w = (const uint16_t*)((const uint8_t*)W + r * ldw);
        for (int c = 0; c < cols; c++) mx = std::max(mx, std::fabs(bf2f(w[c])));
    }
    *quant = 127 / mx; *dequant = mx / 127;
    for (int r = 0; r < rows; r++) {
        const uint16_t* w = (const uint16_t*)((const uint8_t*)W + r * ldw);
        for (int c = 0; c < cols; c++) Wq[(size_t)r * cols + c] = f2s8(bf2f(w[c]) * *quant);
    }
}

// fp32 accumulators of bf16 A x int8 weights: the int8 values are widened to bf16 exactly
// (i8_to_bf16_Kx32, include/kernels_amx.hpp:490-506) and multiplied like orc_gemm_bf16.
void orc_gemm_bf16_w8(const uint16_t* A, int64_t lda, const int8_t* Wq, int64_t ldw, int transposeB, int M, int K, int N,
                      float* acc, int64_t ld_acc_elems) {
    int rows = transposeB ? N : K, cols = transposeB ? K : N;
    std::vector<uint16_t> Wb((size_t)rows * cols);
    for (int r = 0; r < rows; r++)
        for (int c = 0; c < cols; c++) Wb[(size_t)r * cols + c] = f2bf((float)Wq[r * ldw + c]);
    orc_gemm_bf16(A, lda, Wb.data(), (int64_t)cols * 2, transposeB, M, K, N, acc, ld_acc_elems);
}

// MatmulVector / GemAvB (include/kernels_amx.hpp:833-1043, 1529-1618): c[m] = sum_k A[m,k] * b[k]; the intended full
// dot product (the reference's 5- and 6-tile branches are defective and untested; parity is claimed for K <= 4 tiles).
void orc_matvec_bf16(const uint16_t* A, int64_t lda, int M, int K, const uint16_t* b, float* c) {
    #pragma omp parallel for
    for (int m = 0; m < M; m++) {
        const uint16_t* a = (const uint16_t*)((const uint8_t*)A + m * lda);
        float s = 0.0f;
        for (int k = 0; k < K; k++) s = s + bf2f(a[k]) * bf2f(b[k]);
        c[m] = s;
    }
}
void orc_matvec_s8(const int8_t* A, int64_t lda, int M, int K, const int8_t* b, int32_t* c) {
    #pragma omp parallel for
    for (int m = 0; m < M; m++) {
        const int8_t* a = A + m * lda;
        int32_t s = 0;
        for (int k = 0; k < K; k++) s += (int32_t)a[k] * (int32_t)b[k];
        c[m] = s;
    }
}

// Fused Llama MLP, AMX_MLP::MLP::run (tests/amx-mlp.cpp:778-783): x[M,K] bf16; gate, up [N,K] and down [K,N] in
// torch nn.Linear layout.  act = bf16(silu(x gate^T) * (x up^T)) (runGateUp, :707-737); the down projection is
// two fp32 partial sums over the K halves [0, ceil(nblk/2)*256) and the rest, added in fp32 and rounded to bf16
// (Linear::setup :559-589, run :656-683).  act_out (optional) receives the [M,N] bf16 intermediate.
// partial_out (optional) receives the fp32 sum before rounding: a tensor-parallel rank's contribution when the
// weights passed in are that rank's slice of the N (intermediate) dimension; out may then be null.
void orc_mlp(const uint16_t* x, int64_t ldx, int M, const uint16_t* gate, const uint16_t* up, const uint16_t* down,
             int K, int N, uint16_t* out, int64_t ldo, uint16_t* act_out, float* partial_out) {
    std::vector<float> g((size_t)M * N), u((size_t)M * N);
    orc_gemm_bf16(x, ldx, gate, (int64_t)K * 2, 1, M, K, N, g.data(), N);
    orc_gemm_bf16(x, ldx, up, (int64_t)K * 2, 1, M, K, N, u.data(), N);
    std::vector<uint16_t> act((size_t)M * N);
    #pragma omp parallel for
    for (int64_t i = 0; i < (int64_t)M * N; i++) act[i] = f2bf(silu(g[i]) * u[i]);
    if (act_out) memcpy(act_out, act.data(), sizeof(uint16_t) * (size_t)M * N);
    int nblk = (N + 255) / 256;
    int k0 = std::min(N, ((nblk + 1) / 2) * 256), k1 = N - k0;
    std::vector<float> p0((size_t)M * K), p1((size_t)M * K, 0.0f);
    orc_gemm_bf16(act.data(), (int64_t)N * 2, down, (int64_t)N * 2, 1, M, k0, K, p0.data(), K);
    if (k1 > 0) orc_gemm_bf16(act.data() + k0, (int64_t)N * 2, down + k0, (int64_t)N * 2, 1, M, k1, K, p1.data(), K);
    #pragma omp parallel for
    for (int m = 0; m < M; m++)
        for (int j = 0; j < K; j++) {
            float v = p0[(size_t)m * K + j] + p1[(size_t)m * K + j];
            if (partial_out) partial_out[(size_t)m * K + j] = v;
            if (out) ((uint16_t*)((uint8_t*)out + m * ldo))[j] = f2bf(v);
        }
}

}  // extern "C"
