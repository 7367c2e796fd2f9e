// TEST INFRASTRUCTURE — not part of the shipped library.
//
// C-ABI shim around the reference's own CPU kernels (usstq/mm_amx, include/kernels_amx.hpp).  The reference
// header is compiled where it lies (-I<reference>/include); nothing of it is copied.  The resulting shared
// object is used (a) to pin the plain-C++ oracle port against the real AMX implementation and to generate the
// golden fixtures, and (b) as the "reference" CPU arm of the benchmark on hosts whose CPU has AMX.
//
// Needs a CPU with amx_tile/amx_bf16/amx_int8 + avx512_bf16.  Build: see oracle/Makefile (target _ref).
//
// Reference entry points wrapped here (file:line in the reference tree):
//   amx_kernel::Matmul<TA,TB,TC>::operator()            include/kernels_amx.hpp:1169-1314
//   amx_kernel::Matmul<bf16,int8_t,float>::operator()   include/kernels_amx.hpp:1343-1516
//   amx_kernel::PP::BiasGeluStore                       include/kernels_amx.hpp:552-673
//   amx_kernel::MatmulVector / GemAvB                   include/kernels_amx.hpp:833-1043, 1529-1618
//   N-split over threads like MatmulMTOMP               main.cpp:442-479
//   fused MLP arithmetic (gate/up interleave, SiLU*up, 2-way split-K down)  tests/amx-mlp.cpp:545-783
//     — that file needs xbyak (absent), so its arithmetic is restated here around the reference Matmul.
#include <immintrin.h>
#include <cstdint>
#include <cstring>
#include <vector>
#include <memory>
#include <algorithm>
#include <omp.h>

// GCC spells _tile_zero as a macro that pastes its operand into the asm text, which breaks when the operand is a
// template parameter (the reference targets icpx).  Route it through a constant-folded switch instead.
#undef _tile_zero
static inline __attribute__((always_inline)) void harness_tile_zero(int t) {
    switch (t) {
        case 0: __asm__ volatile("tilezero %%tmm0" ::); break;
        case 1: __asm__ volatile("tilezero %%tmm1" ::); break;
        case 2: __asm__ volatile("tilezero %%tmm2" ::); break;
        case 3: __asm__ volatile("tilezero %%tmm3" ::); break;
        case 4: __asm__ volatile("tilezero %%tmm4" ::); break;
        case 5: __asm__ volatile("tilezero %%tmm5" ::); break;
        case 6: __asm__ volatile("tilezero %%tmm6" ::); break;
        case 7: __asm__ volatile("tilezero %%tmm7" ::); break;
    }
}
#define _tile_zero(t) harness_tile_zero(t)

#include "kernels_amx.hpp"

using bf16 = ov::bfloat16;
namespace PP = amx_kernel::PP;

namespace {

inline uint16_t bits_of(bf16 b) { uint16_t u; memcpy(&u, &b, 2); return u; }

// ---- functors written for the harness (allowed by the reference's functor contract, kernels_amx.hpp:1074-1091) --
// raw copy of the accumulator block (bit-exact int32 / fp32 accumulators)
template <typename T>
struct RawStore {
    T* C; int ldc;  // elements
    void set_deq_scale(float) {}
    void operator()(tensor2D<T>& buffC, int m, int n, int valid_m, int valid_n) {
        for (int i = 0; i < valid_m; i++)
            memcpy(C + (size_t)(m + i) * ldc + n, &buffC(i, 0), sizeof(T) * valid_n);
    }
};

// fp32 accumulator * scale[n] (+ bias[n]) -> bf16 RNE; used for the per-output-channel int8-weight decode config
struct PerChannelStore {
    uint16_t* C; int ldc; const float* scale; const float* bias;
    float tensor_scale = 1.0f;
    void set_deq_scale(float s) { tensor_scale = s; }
    void operator()(tensor2D<float>& buffC, int m, int n, int valid_m, int valid_n) {
        for (int i = 0; i < valid_m; i++)
            for (int j = 0; j < valid_n; j++) {
                float v = buffC(i, j) * tensor_scale;
                v *= scale[n + j];
                if (bias) v += bias[n + j];
                C[(size_t)(m + i) * ldc + n + j] = bits_of(bf16(v));
            }
    }
};

// exp / SiLU of tests/amx-mlp.cpp:383-456 restated with the same operation sequence (clamp, n = floor(x*log2e+.5),
// degree-5 polynomial on the remainder, 2 * 2^(n-1) scaling, rcp14 reciprocal).
inline __m512 bits512(uint32_t u) { return _mm512_castsi512_ps(_mm512_set1_epi32((int)u)); }
inline __m512 harness_exp(__m512 x) {
    const __m512 lo = bits512(0xc2aeac50), hi = bits512(0x42b17218);
    __mmask16 under = _mm512_cmp_ps_mask(x, lo, _CMP_LT_OS);
    x = _mm512_max_ps(_mm512_min_ps(x, hi), lo);
    __m512 n = _mm512_floor_ps(_mm512_add_ps(_mm512_mul_ps(x, bits512(0x3fb8aa3b)), bits512(0x3f000000)));
    __m512 r = _mm512_fnmadd_ps(n, bits512(0x3f317218), x);
    __m512i e = _mm512_cvtps_epi32(_mm512_sub_ps(n, _mm512_set1_ps(1.0f)));
    e = _mm512_slli_epi32(_mm512_add_epi32(e, _mm512_set1_epi32(127)), 23);
    __m512 scale = _mm512_mask_blend_ps(under, _mm512_castsi512_ps(e), _mm512_setzero_ps());
    __m512 p = bits512(0x3c07cfce);
    p = _mm512_fmadd_ps(p, r, bits512(0x3d2b9d0d));
    p = _mm512_fmadd_ps(p, r, bits512(0x3e2aad40));
    p = _mm512_fmadd_ps(p, r, bits512(0x3efffee3));
    p = _mm512_fmadd_ps(p, r, bits512(0x3f7ffffb));
    p = _mm512_fmadd_ps(p, r, _mm512_set1_ps(1.0f));
    return _mm512_mul_ps(_mm512_mul_ps(p, scale), _mm512_set1_ps(2.0f));
}
inline __m512 harness_silu(__m512 x) {
    __m512 e = harness_exp(_mm512_sub_ps(_mm512_setzero_ps(), x));
    return _mm512_mul_ps(x, _mm512_rcp14_ps(_mm512_add_ps(_mm512_set1_ps(1.0f), e)));
}

// gate/up epilogue of tests/amx-mlp.cpp:716-734: columns [0,16) = gate, [16,32) = up of the same 16 channels
struct SiluMulStore {
    uint16_t* act; int ld;  // elements
    void operator()(tensor2D<float>& buffC, int m, int n, int valid_m, int valid_n) {
        (void)valid_n;
        for (int i = 0; i < valid_m; i++) {
            __m512 g = _mm512_loadu_ps(&buffC(i, 0));
            __m512 u = _mm512_loadu_ps(&buffC(i, 16));
            __m256bh o = _mm512_cvtneps_pbh(_mm512_mul_ps(harness_silu(g), u));
            _mm256_storeu_si256((__m256i*)(act + (size_t)(m + i) * ld + n / 2), (__m256i)o);
        }
    }
};

template <typename T>
tensor2D<T> view(const void* p, int d0, int d1, int stride_bytes) {
    return tensor2D<T>(d0, d1, reinterpret_cast<T*>(const_cast<void*>(p)), stride_bytes);
}

struct Range { int n0, n1; };
inline Range thread_cols(int N, int nthr, int tid) {
    // 32-column work units, as MatmulMTOMP does (main.cpp:453-478)
    int units = (N + 31) / 32, s, e;
    splitter(units, nthr, tid, s, e);
    return {std::min(s * 32, N), std::min(e * 32, N)};
}

enum Kind { K_BF16 = 0, K_S8 = 1, K_W8 = 2 };

struct FC {
    int kind, nthr;
    bool transposeB;
    std::vector<amx_kernel::Matmul<bf16, bf16>> mm_bf16;
    std::vector<amx_kernel::Matmul<int8_t, int8_t>> mm_s8;
    std::vector<amx_kernel::Matmul<bf16, int8_t, float>> mm_w8;
};

template <typename D, int STEPS, typename MM, typename TA, typename TB>
void run_pp(std::vector<MM>& ops, int nthr, tensor2D<TA>& A, tensor2D<TB>& B, int N, tensor2D<D>& C,
            float* bias, float deq, float q, float* q_oc) {
    PP::BiasGeluStore<D, (PP::Steps)STEPS> pp(C, bias);
    if (STEPS & PP::DEQUANT) pp.set_deq_scale(deq);
    if (STEPS & PP::QUANT) { if (q_oc) pp.set_q_scale(q_oc); else pp.set_q_scale(q); }
    #pragma omp parallel num_threads(nthr)
    {
        int tid = omp_get_thread_num();
        Range r = thread_cols(N, nthr, tid);
        if (r.n1 > r.n0) ops[tid](A, B, r.n0, r.n1, pp);
    }
}

template <typename D, typename MM, typename TA, typename TB>
int dispatch_steps(int steps, std::vector<MM>& ops, int nthr, tensor2D<TA>& A, tensor2D<TB>& B, int N,
                   tensor2D<D>& C, float* bias, float deq, float q, float* q_oc) {
    switch (steps) {
#define CASE(S) case S: run_pp<D, S>(ops, nthr, A, B, N, C, bias, deq, q, q_oc); return 0;
        CASE(0) CASE(1) CASE(2) CASE(3) CASE(4) CASE(5) CASE(6) CASE(7)
        CASE(8) CASE(9) CASE(10) CASE(11) CASE(12) CASE(13) CASE(14) CASE(15)
#undef CASE
    }
    return -1;
}

template <typename MM, typename TA, typename TB>
int dispatch_out(int out_dtype, int steps, std::vector<MM>& ops, int nthr, tensor2D<TA>& A, tensor2D<TB>& B, int M,
                 int N, void* C, int ldc_bytes, float* bias, float deq, float q, float* q_oc) {
    if (out_dtype == 0) { auto c = view<float>(C, M, N, ldc_bytes);  return dispatch_steps<float>(steps, ops, nthr, A, B, N, c, bias, deq, q, q_oc); }
    if (out_dtype == 1) { auto c = view<bf16>(C, M, N, ldc_bytes);   return dispatch_steps<bf16>(steps, ops, nthr, A, B, N, c, bias, deq, q, q_oc); }
    if (out_dtype == 2) { auto c = view<int8_t>(C, M, N, ldc_bytes); return dispatch_steps<int8_t>(steps, ops, nthr, A, B, N, c, bias, deq, q, q_oc); }
    return -1;
}

struct MLP {
    int K, N, nthr;                       // K = hidden, N = intermediate
    std::vector<uint16_t> w_gate_up;      // [2N, K], rows interleaved 16 gate / 16 up (tests/amx-mlp.cpp:758-765)
    const uint16_t* w_down;               // [K, N] as given
    int k_split;                          // first K-half length of the down projection (tests/amx-mlp.cpp:559-589)
    std::vector<amx_kernel::Matmul<bf16, bf16>> gu, d0, d1;
    std::vector<uint16_t> act;
    std::vector<float> p0, p1;
};

}  // namespace

extern "C" {

int ref_init() { return initXTILE() ? 0 : -1; }
int ref_max_threads() { return omp_get_max_threads(); }

void* ref_fc_create(int kind, int constB, int transposeB, int nthr) {
    FC* f = new FC;
    f->kind = kind; f->nthr = nthr; f->transposeB = transposeB != 0;
    for (int i = 0; i < nthr; i++) {
        if (kind == K_BF16) f->mm_bf16.emplace_back(constB != 0, transposeB != 0);
        if (kind == K_S8) f->mm_s8.emplace_back(constB != 0, transposeB != 0);
        if (kind == K_W8) f->mm_w8.emplace_back(constB != 0, transposeB != 0);
    }
    return f;
}
void ref_fc_free(void* h) { delete (FC*)h; }

// C = BiasGeluStore<D, steps>(A * B).  B is [K,N] (or [N,K] when the handle was made with transposeB).
// out_dtype: 0 fp32, 1 bf16, 2 int8.  For kind K_W8 A and B are bf16 and DEQUANT must be in steps.
int ref_fc_run(void* h, const void* A, int lda_bytes, const void* B, int ldb_bytes, int M, int K, int N, int steps,
               float* bias, float deq_scale, float q_scale, float* q_scale_per_oc, int out_dtype, void* C,
               int ldc_bytes) {
    FC* f = (FC*)h;
    int bd0 = f->transposeB ? N : K, bd1 = f->transposeB ? K : N;
    if (f->kind == K_S8) {
        auto a = view<int8_t>(A, M, K, lda_bytes); auto b = view<int8_t>(B, bd0, bd1, ldb_bytes);
        return dispatch_out(out_dtype, steps, f->mm_s8, f->nthr, a, b, M, N, C, ldc_bytes, bias, deq_scale, q_scale, q_scale_per_oc);
    }
    auto a = view<bf16>(A, M, K, lda_bytes); auto b = view<bf16>(B, bd0, bd1, ldb_bytes);
    if (f->kind == K_BF16)
        return dispatch_out(out_dtype, steps, f->mm_bf16, f->nthr, a, b, M, N, C, ldc_bytes, bias, deq_scale, q_scale, q_scale_per_oc);
    if (!(steps & PP::DEQUANT)) return -2;
    return dispatch_out(out_dtype, steps, f->mm_w8, f->nthr, a, b, M, N, C, ldc_bytes, bias, deq_scale, q_scale, q_scale_per_oc);
}

// raw accumulators (int32 for K_S8, fp32 for K_BF16): the bit-exact view of the tile results
int ref_fc_run_raw(void* h, const void* A, int lda_bytes, const void* B, int ldb_bytes, int M, int K, int N, void* C,
                   int ldc_elems) {
    FC* f = (FC*)h;
    int bd0 = f->transposeB ? N : K, bd1 = f->transposeB ? K : N;
    if (f->kind == K_S8) {
        auto a = view<int8_t>(A, M, K, lda_bytes); auto b = view<int8_t>(B, bd0, bd1, ldb_bytes);
        RawStore<int32_t> pp{(int32_t*)C, ldc_elems};
        #pragma omp parallel num_threads(f->nthr)
        { Range r = thread_cols(N, f->nthr, omp_get_thread_num()); if (r.n1 > r.n0) f->mm_s8[omp_get_thread_num()](a, b, r.n0, r.n1, pp); }
        return 0;
    }
    if (f->kind == K_BF16) {
        auto a = view<bf16>(A, M, K, lda_bytes); auto b = view<bf16>(B, bd0, bd1, ldb_bytes);
        RawStore<float> pp{(float*)C, ldc_elems};
        #pragma omp parallel num_threads(f->nthr)
        { Range r = thread_cols(N, f->nthr, omp_get_thread_num()); if (r.n1 > r.n0) f->mm_bf16[omp_get_thread_num()](a, b, r.n0, r.n1, pp); }
        return 0;
    }
    return -1;
}

// int8-compressed weights with a per-output-channel scale.  B holds integer-valued bf16 weights whose absmax is
// 127, so the reference's per-tensor quantiser (kernels_amx.hpp:1363-1377) reproduces them exactly as int8 and
// hands the functor a tensor scale of 1; the per-channel scale (and optional bias) is applied in the functor.
int ref_fc_run_w8_per_channel(void* h, const void* A, int lda_bytes, const void* B, int ldb_bytes, int M, int K, int N,
                              const float* scale, const float* bias, uint16_t* C, int ldc_elems) {
    FC* f = (FC*)h;
    if (f->kind != K_W8) return -1;
    int bd0 = f->transposeB ? N : K, bd1 = f->transposeB ? K : N;
    auto a = view<bf16>(A, M, K, lda_bytes); auto b = view<bf16>(B, bd0, bd1, ldb_bytes);
    PerChannelStore pp{C, ldc_elems, scale, bias};
    #pragma omp parallel num_threads(f->nthr)
    { Range r = thread_cols(N, f->nthr, omp_get_thread_num()); if (r.n1 > r.n0) f->mm_w8[omp_get_thread_num()](a, b, r.n0, r.n1, pp); }
    return 0;
}

// the quantised weights the compressed path holds after its first call (for checking the GPU packer), returned
// as scale only: quant = 127/absmax, dequant = absmax/127
int ref_fc_w8_scales(void* h, float* quant, float* dequant) {
    FC* f = (FC*)h;
    if (f->kind != K_W8 || f->mm_w8.empty()) return -1;
    *quant = f->mm_w8[0].quant_scale_B; *dequant = f->mm_w8[0].dequant_scale_B;
    return 0;
}

int ref_matvec_bf16(const void* A, int lda_bytes, int M, int K, const void* b, float* c) {
    auto a = view<bf16>(A, M, K, lda_bytes);
    amx_kernel::MatmulVector<bf16, bf16> mv;
    mv(a, (const bf16*)b, c);
    return 0;
}
int ref_matvec_s8(const void* A, int lda_bytes, int M, int K, const void* b, int32_t* c) {
    auto a = view<int8_t>(A, M, K, lda_bytes);
    amx_kernel::MatmulVector<int8_t, int8_t> mv;
    mv(a, (const int8_t*)b, c);
    return 0;
}
int ref_gemavb(const void* A, int lda_bytes, int M, int K, void* b, float* c) {
    auto a = view<bf16>(A, M, K, lda_bytes);
    amx_kernel::GemAvB g;
    g(a, (bf16*)b, c);
    return 0;
}

void ref_gelu(const float* x, float* y, int n) {  // n multiple of 16
    for (int i = 0; i < n; i += 16) {
        __m512 v = _mm512_loadu_ps(x + i);
        _mm512_storeu_ps(y + i, amx_kernel::functional::gelu_erf_minmax_approx(v));
    }
}
void ref_silu(const float* x, float* y, int n) {  // n multiple of 16
    for (int i = 0; i < n; i += 16) _mm512_storeu_ps(y + i, harness_silu(_mm512_loadu_ps(x + i)));
}

// ---- fused Llama MLP: gate/up [N,K], down [K,N] in torch nn.Linear layout, all bf16 contiguous ----
void* ref_mlp_create(const uint16_t* gate, const uint16_t* up, const uint16_t* down, int K, int N, int nthr) {
    if (N % 32 || K % 256 || N % 256) return nullptr;
    MLP* m = new MLP;
    m->K = K; m->N = N; m->nthr = nthr; m->w_down = down;
    m->w_gate_up.resize((size_t)2 * N * K);
    for (int n = 0; n < N; n += 16) {
        memcpy(&m->w_gate_up[(size_t)(2 * n) * K], gate + (size_t)n * K, sizeof(uint16_t) * 16 * K);
        memcpy(&m->w_gate_up[(size_t)(2 * n + 16) * K], up + (size_t)n * K, sizeof(uint16_t) * 16 * K);
    }
    int nblk = N / 256;
    m->k_split = ((nblk + 1) / 2) * 256;
    for (int i = 0; i < nthr; i++) {
        m->gu.emplace_back(true, true); m->d0.emplace_back(true, true); m->d1.emplace_back(true, true);
    }
    return m;
}
void ref_mlp_free(void* h) { delete (MLP*)h; }

int ref_mlp_run(void* h, const uint16_t* x, int ldx_bytes, int M, uint16_t* out, int ldo_bytes) {
    MLP* m = (MLP*)h;
    int K = m->K, N = m->N, nthr = m->nthr;
    m->act.resize((size_t)M * N); m->p0.resize((size_t)M * K); m->p1.resize((size_t)M * K);
    auto A = view<bf16>(x, M, K, ldx_bytes);
    auto Wgu = view<bf16>(m->w_gate_up.data(), 2 * N, K, K * 2);
    SiluMulStore pp{m->act.data(), N};
    #pragma omp parallel num_threads(nthr)
    { int t = omp_get_thread_num(); Range r = thread_cols(2 * N, nthr, t); if (r.n1 > r.n0) m->gu[t](A, Wgu, r.n0, r.n1, pp); }
    int k0 = m->k_split, k1 = N - k0;
    auto A0 = view<bf16>(m->act.data(), M, k0, N * 2);
    auto A1 = view<bf16>(m->act.data() + k0, M, k1, N * 2);
    auto W0 = view<bf16>(m->w_down, K, k0, N * 2);
    auto W1 = view<bf16>(m->w_down + k0, K, k1, N * 2);
    RawStore<float> s0{m->p0.data(), K}, s1{m->p1.data(), K};
    #pragma omp parallel num_threads(nthr)
    {
        int t = omp_get_thread_num(); Range r = thread_cols(K, nthr, t);
        if (r.n1 > r.n0) { m->d0[t](A0, W0, r.n0, r.n1, s0); if (k1 > 0) m->d1[t](A1, W1, r.n0, r.n1, s1); }
    }
    #pragma omp parallel for num_threads(nthr)
    for (int i = 0; i < M; i++) {
        uint16_t* o = (uint16_t*)((uint8_t*)out + (size_t)i * ldo_bytes);
        for (int j = 0; j < K; j++) {
            float v = m->p0[(size_t)i * K + j] + (k1 > 0 ? m->p1[(size_t)i * K + j] : 0.0f);
            o[j] = bits_of(bf16(v));
        }
    }
    return 0;
}
// intermediate activation of the last run ([M, N] bf16), for layer-by-layer checks
const uint16_t* ref_mlp_act(void* h) { return ((MLP*)h)->act.data(); }

}  // extern "C"
