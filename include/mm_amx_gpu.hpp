// Header-only C++ façade over the b200fc C ABI with the class names, constructor flags and call signatures of
// usstq/mm_amx, so code written against the reference's headers can switch to the GPU by changing an #include.
//
//   reference                                            here
//   ov::bfloat16            include/bf16.hpp             ov::bfloat16          (same 16-bit layout, RNE conversion)
//   tensor2D<T>             include/tensor2D.hpp:30-330  tensor2D<T>           (host memory; same fields / accessors)
//   amx_kernel::PP::Steps, PP::BiasGeluStore             amx_kernel::PP::...   (include/kernels_amx.hpp:540-673)
//   amx_kernel::Matmul<TA,TB,TC>(constB, transposeB)     amx_kernel::Matmul    (kernels_amx.hpp:1045-1314, 1319-1516)
//   amx_kernel::MatmulVector, GemAvB                     same names            (kernels_amx.hpp:833-1043, 1529-1618)
//   AMX_MLP::MLP::setup / run                            AMX_MLP::MLP          (tests/amx-mlp.cpp:740-784)
//
// Tensors live in host memory exactly as in the reference; every call stages its operands through the library's
// `_host` entry points (weights are packed to the GPU once when constB is set, as the reference caches internalB).
// Arbitrary host callables cannot run in a GPU epilogue: the post-op argument must be a PP::BiasGeluStore.
// Errors throw std::runtime_error with the library's message (the reference asserts / aborts).
// Link with -lb200fc (mm_amx_b200/libb200fc.so).
#pragma once
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <cmath>
#include <memory>
#include <stdexcept>
#include <string>
#include <type_traits>
#include "b200fc.h"

namespace ov {
// 16-bit brain float: the upper half of an IEEE binary32, converted with round-to-nearest-even
class bfloat16 {
public:
    bfloat16() : bits_(0) {}
    bfloat16(float v) : bits_(round_bits(v)) {}
    template <typename I, typename = typename std::enable_if<std::is_integral<I>::value>::type>
    explicit bfloat16(I v) : bits_(round_bits(static_cast<float>(v))) {}
    operator float() const {
        uint32_t u = static_cast<uint32_t>(bits_) << 16;
        float f;
        std::memcpy(&f, &u, sizeof f);
        return f;
    }
    static bfloat16 from_bits(uint16_t b) { bfloat16 r; r.bits_ = b; return r; }
    uint16_t to_bits() const { return bits_; }

private:
    static uint16_t round_bits(float v) {
        uint32_t u;
        std::memcpy(&u, &v, sizeof u);
        if ((u & 0x7f800000u) == 0x7f800000u) return static_cast<uint16_t>((u >> 16) | ((u & 0x7fffffu) ? 0x40 : 0));
        return static_cast<uint16_t>((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
    }
    uint16_t bits_;
};
}  // namespace ov

namespace b200fc_detail {
inline void check(int rc) {
    if (rc != B200FC_OK) throw std::runtime_error(std::string("b200fc: ") + b200fc_last_error());
}
template <typename T> struct dtype_of;
template <> struct dtype_of<ov::bfloat16> { static constexpr int value = B200FC_BF16; };
template <> struct dtype_of<int8_t> { static constexpr int value = B200FC_S8; };
template <> struct dtype_of<uint8_t> { static constexpr int value = B200FC_U8; };
template <> struct dtype_of<float> { static constexpr int value = B200FC_F32; };
template <> struct dtype_of<int32_t> { static constexpr int value = B200FC_S32; };
inline int round_up(int v, int m) { return (v + m - 1) / m * m; }
}  // namespace b200fc_detail

// 2-D host tensor: dims, shared data pointer, byte stride (rows padded to 64 bytes unless force_compact), element
// accessors — the members callers of the reference rely on.
template <typename T>
struct tensor2D {
    int dims[2] = {0, 0};
    std::shared_ptr<T> data;
    uint64_t capacity = 0;
    int stride = 0;
    bool force_compact = false;
    int padded_dim1 = 0;

    tensor2D() = default;
    tensor2D(int d0, int d1, bool compact = false) { resize(d0, d1, compact); fill_rnd(); }
    // non-owning view of external memory with a byte stride
    tensor2D(int d0, int d1, T* ext, int stride_bytes) {
        capacity = 1;
        data = std::shared_ptr<T>(ext, [](T*) {});
        dims[0] = d0; dims[1] = d1;
        stride = stride_bytes;
        padded_dim1 = stride / static_cast<int>(sizeof(T));
    }
    explicit operator bool() const { return dims[0] * dims[1] > 0; }

    void resize(int d0, int d1, bool compact = false) {
        force_compact = compact;
        dims[0] = d0; dims[1] = d1;
        stride = d1 * static_cast<int>(sizeof(T));
        if (!compact) stride = b200fc_detail::round_up(stride, 64);
        padded_dim1 = stride / static_cast<int>(sizeof(T));
        uint64_t need = static_cast<uint64_t>(d0) * stride + 64;
        if (capacity < need) {
            void* p = nullptr;
            if (posix_memalign(&p, 64, need) != 0) throw std::bad_alloc();
            std::memset(p, 0, need);
            data = std::shared_ptr<T>(static_cast<T*>(p), [](T* q) { std::free(q); });
            capacity = need;
        }
    }
    T& operator[](int i) { return data.get()[i]; }
    const T& operator[](int i) const { return data.get()[i]; }
    T& operator()(int r, int c) { return data.get()[static_cast<int64_t>(r) * padded_dim1 + c]; }
    const T& operator()(int r, int c) const { return data.get()[static_cast<int64_t>(r) * padded_dim1 + c]; }

    // two-valued random fill like the reference's test data: +-0.5 for float types, +-1 for integers
    void fill_rnd() {
        for (int r = 0; r < dims[0]; r++)
            for (int c = 0; c < dims[1]; c++) {
                bool neg = (std::rand() & 1) != 0;
                if (std::is_integral<T>::value) (*this)(r, c) = static_cast<T>(neg ? -1 : 1);
                else (*this)(r, c) = static_cast<T>(neg ? -0.5f : 0.5f);
            }
    }
    tensor2D<T>& operator=(const T& v) {
        for (int r = 0; r < dims[0]; r++)
            for (int c = 0; c < dims[1]; c++) (*this)(r, c) = v;
        return *this;
    }
    tensor2D<T> Tr() const {
        tensor2D<T> t;
        t.resize(dims[1], dims[0]);
        for (int r = 0; r < dims[0]; r++)
            for (int c = 0; c < dims[1]; c++) t(c, r) = (*this)(r, c);
        return t;
    }
    tensor2D<T> clone() const {
        tensor2D<T> t;
        t.resize(dims[0], dims[1], force_compact);
        for (int r = 0; r < dims[0]; r++) std::memcpy(&t(r, 0), &(*this)(r, 0), sizeof(T) * dims[1]);
        return t;
    }
    // element-wise closeness with the reference's defaults (rtol 1e-5, atol 1e-8); NaN never matches
    bool allclose(const tensor2D<T>& o, float rtol = 1e-5f, float atol = 1e-8f) const {
        if (dims[0] != o.dims[0] || dims[1] != o.dims[1]) return false;
        for (int r = 0; r < dims[0]; r++)
            for (int c = 0; c < dims[1]; c++) {
                float a = static_cast<float>((*this)(r, c)), b = static_cast<float>(o(r, c));
                if (!(std::fabs(a - b) <= atol + rtol * std::fabs(b))) return false;
            }
        return true;
    }
    bool operator==(const tensor2D<T>& o) const { return allclose(o); }
};

namespace amx_kernel {

namespace PP {
enum Steps {
    NONE = 0,
    DEQUANT = 1 << 0,
    BIAS = 1 << 1,
    GELU = 1 << 2,
    QUANT = 1 << 3,
    BIAS_GELU = BIAS | GELU,
    DEQUANT_BIAS_GELU = DEQUANT | BIAS_GELU,
    DEQUANT_BIAS_GELU_QUANT = DEQUANT_BIAS_GELU | QUANT
};

// Captures the output tensor and the post-op parameters; the GPU epilogue executes the steps in the reference's
// order: [int32 -> fp32] -> DEQUANT -> BIAS -> GELU -> QUANT -> store as D.
template <typename D, Steps steps>
struct BiasGeluStore {
    static_assert(std::is_same<D, ov::bfloat16>::value || std::is_same<D, int8_t>::value || std::is_same<D, float>::value,
                  "BiasGeluStore supports ov::bfloat16 / int8_t / float outputs");
    static constexpr Steps kSteps = steps;
    using out_type = D;
    BiasGeluStore(tensor2D<D>& C, float* bias = nullptr) : C(C), bias(bias) {}
    tensor2D<D>& C;
    float* bias;
    float deq_scale = 1.0f;
    float q_scale_common = 0.0f;
    float* q_scale_per_oc = nullptr;
    void set_bias(float* b) { bias = b; }
    void set_deq_scale(float s = 1.0f) { deq_scale = s; }
    void set_q_scale(float s) { q_scale_common = s; q_scale_per_oc = nullptr; }
    void set_q_scale(float* per_oc) { q_scale_common = 0; q_scale_per_oc = per_oc; }

    b200fc_epilogue_t descriptor() const {
        b200fc_epilogue_t ep;
        std::memset(&ep, 0, sizeof ep);
        ep.steps = steps;
        ep.out_dtype = b200fc_detail::dtype_of<D>::value;
        ep.C = &C[0];               // column indices are global, like the reference functor's (m, n)
        ep.ldc_bytes = C.stride;
        ep.bias = bias;
        ep.deq_scale = deq_scale;
        ep.q_scale = q_scale_common;
        ep.q_scale_per_oc = q_scale_per_oc;
        return ep;
    }
};
}  // namespace PP

template <typename T> struct acc_type { using type = float; };
template <> struct acc_type<int8_t> { using type = int32_t; };
template <> struct acc_type<uint8_t> { using type = int32_t; };

namespace detail {
// Packed weights on the GPU for the column range a Matmul object was first called with (the reference packs the
// sub-matrix [n0, n1) into internalB; one object per thread holds one range).
struct PackedRange {
    b200fc_weight_t* w = nullptr;
    int n0 = 0, n1 = 0;
    ~PackedRange() { b200fc_weight_free(w); }
    PackedRange() = default;
    PackedRange(const PackedRange&) = delete;
    PackedRange& operator=(const PackedRange&) = delete;
    void reset() { b200fc_weight_free(w); w = nullptr; }
};

template <typename TA, typename TB, int PACK_MODE>
struct MatmulImpl {
    bool constB, transposeB;
    std::shared_ptr<PackedRange> packed = std::make_shared<PackedRange>();
    MatmulImpl(bool constB, bool transposeB) : constB(constB), transposeB(transposeB) {}

    template <typename PPK>
    void run(tensor2D<TA>& A, tensor2D<TB>& B, int n0, int n1, PPK pp) {
        using b200fc_detail::check;
        const int M = A.dims[0], K = A.dims[1];
        const int Nfull = B.dims[transposeB ? 0 : 1];
        if (K != B.dims[transposeB ? 1 : 0]) throw std::runtime_error("Matmul: K of A and B differ");
        if (n0 < 0 || n1 > Nfull || n0 > n1) throw std::runtime_error("Matmul: bad column range");
        PackedRange& pr = *packed;
        if (!constB || !pr.w || pr.n0 != n0 || pr.n1 != n1) {
            pr.reset();
            // view of the columns [n0, n1): rows n0.. of an [N, K] matrix, or a column offset into a [K, N] one
            const TB* base = transposeB ? &B(n0, 0) : &B(0, n0);
            float absmax = 0.0f;
            const float* scales = nullptr;
            if (PACK_MODE == B200FC_PACK_QUANT_TENSOR) {
                // the quantisation scale comes from the WHOLE weight matrix, whatever range this object computes
                for (int r = 0; r < B.dims[0]; r++)
                    for (int c = 0; c < B.dims[1]; c++) absmax = std::fmax(absmax, std::fabs(static_cast<float>(B(r, c))));
                scales = &absmax;
            }
            check(b200fc_weight_pack(base, b200fc_detail::dtype_of<TB>::value, K, n1 - n0, B.stride, transposeB ? 1 : 0,
                                     PACK_MODE, scales, &pr.w, nullptr));
            pr.n0 = n0; pr.n1 = n1;
        }
        b200fc_epilogue_t ep = pp.descriptor();
        // the packed object covers columns [n0, n1) as [0, n1 - n0): shift the column-indexed arrays accordingly
        using D = typename PPK::out_type;
        ep.C = reinterpret_cast<char*>(ep.C) + static_cast<int64_t>(n0) * sizeof(D);
        if (ep.bias) ep.bias += n0;
        if (ep.q_scale_per_oc) ep.q_scale_per_oc += n0;
        check(b200fc_matmul_host(pr.w, &A[0], b200fc_detail::dtype_of<TA>::value, M, K, A.stride, 0, n1 - n0, &ep, nullptr));
    }
};
}  // namespace detail

// C[:, n0:n1) = postops(A * B[:, n0:n1)).  constB: B is a weight, packed once; transposeB: B is given as [N, K].
template <typename TA, typename TB, typename TC = typename acc_type<TA>::type>
struct Matmul : detail::MatmulImpl<TA, TB, B200FC_PACK_PLAIN> {
    static_assert((std::is_same<TA, ov::bfloat16>::value && std::is_same<TB, ov::bfloat16>::value) ||
                      ((std::is_same<TA, int8_t>::value || std::is_same<TA, uint8_t>::value) &&
                       (std::is_same<TB, int8_t>::value || std::is_same<TB, uint8_t>::value)),
                  "Matmul supports bf16 x bf16 and 8-bit x 8-bit");
    constexpr static int kStep = std::is_same<TA, ov::bfloat16>::value ? 32 : 64;
    Matmul(bool constB = false, bool transposeB = false) : detail::MatmulImpl<TA, TB, B200FC_PACK_PLAIN>(constB, transposeB) {}
    template <typename PPK>
    void operator()(tensor2D<TA>& A, tensor2D<TB>& B, int n0, int n1, PPK pp) { this->run(A, B, n0, n1, pp); }
    template <typename PPK>
    void operator()(tensor2D<TA>& A, tensor2D<TB>& B, PPK pp) { this->run(A, B, 0, B.dims[this->transposeB ? 0 : 1], pp); }
};

// bf16 activations, bf16 weights stored as int8 with one absmax scale and dequantised on the fly; the weight's scale
// replaces the post-op's deq_scale (the reference calls ppkernel.set_deq_scale(dequant_scale_B)); steps must
// include DEQUANT.  Note: B is still passed as bf16, like the reference.
template <>
struct Matmul<ov::bfloat16, int8_t, float> : detail::MatmulImpl<ov::bfloat16, ov::bfloat16, B200FC_PACK_QUANT_TENSOR> {
    constexpr static int kStep = 32;
    Matmul(bool constB = false, bool transposeB = false)
        : detail::MatmulImpl<ov::bfloat16, ov::bfloat16, B200FC_PACK_QUANT_TENSOR>(constB, transposeB) {}
    template <typename PPK>
    void operator()(tensor2D<ov::bfloat16>& A, tensor2D<ov::bfloat16>& B, int n0, int n1, PPK pp) {
        static_assert((PPK::kSteps & PP::DEQUANT) != 0, "compressed weights need a post-op with the DEQUANT step");
        this->run(A, B, n0, n1, pp);
    }
    template <typename PPK>
    void operator()(tensor2D<ov::bfloat16>& A, tensor2D<ov::bfloat16>& B, PPK pp) {
        (*this)(A, B, 0, B.dims[this->transposeB ? 0 : 1], pp);
    }
};

// bf16 activations, bf16 weights stored as 4-bit values with one absmax scale per output channel and 128 K
// (B200FC_PACK_INT4_GROUP).  The reference reserves this precision in its dispatcher (Weight_INT4, main.cpp:36) without
// implementing it; the tag type stands where int8_t stands in the specialisation above.  Steps must include DEQUANT.
struct int4_t {};
template <>
struct Matmul<ov::bfloat16, int4_t, float> : detail::MatmulImpl<ov::bfloat16, ov::bfloat16, B200FC_PACK_INT4_GROUP> {
    constexpr static int kStep = 32;
    Matmul(bool constB = false, bool transposeB = false)
        : detail::MatmulImpl<ov::bfloat16, ov::bfloat16, B200FC_PACK_INT4_GROUP>(constB, transposeB) {}
    template <typename PPK>
    void operator()(tensor2D<ov::bfloat16>& A, tensor2D<ov::bfloat16>& B, int n0, int n1, PPK pp) {
        static_assert((PPK::kSteps & PP::DEQUANT) != 0, "compressed weights need a post-op with the DEQUANT step");
        this->run(A, B, n0, n1, pp);
    }
    template <typename PPK>
    void operator()(tensor2D<ov::bfloat16>& A, tensor2D<ov::bfloat16>& B, PPK pp) {
        (*this)(A, B, 0, B.dims[this->transposeB ? 0 : 1], pp);
    }
};

// c[M] = A[M, K] * b[K]
template <typename TA, typename TB, typename TC = typename acc_type<TA>::type>
struct MatmulVector {
    static_assert(std::is_same<TA, TB>::value && (std::is_same<TA, ov::bfloat16>::value || std::is_same<TA, int8_t>::value),
                  "MatmulVector supports bf16 x bf16 -> float and int8 x int8 -> int32");
    void operator()(tensor2D<TA>& A, const TB* b, TC* c) {
        b200fc_detail::check(b200fc_matvec_host(&A[0], b200fc_detail::dtype_of<TA>::value, A.dims[0], A.dims[1], A.stride, b,
                                                c, nullptr));
    }
};

struct GemAvB {
    void operator()(tensor2D<ov::bfloat16>& A, ov::bfloat16* b, float* c) {
        b200fc_detail::check(b200fc_matvec_host(&A[0], B200FC_BF16, A.dims[0], A.dims[1], A.stride, b, c, nullptr));
    }
};

}  // namespace amx_kernel

namespace AMX_MLP {
// Fused Llama MLP: out = down(silu(x gate^T) * (x up^T)).  Weights in torch nn.Linear layout: gate, up [N, K],
// down [K, N], bf16 contiguous.
class MLP {
public:
    MLP() = default;
    MLP(const MLP&) = delete;
    MLP& operator=(const MLP&) = delete;
    ~MLP() { b200fc_mlp_free(h_); }
    void setup(ov::bfloat16* w_gate, ov::bfloat16* w_up, ov::bfloat16* w_down, int K, int N) {
        b200fc_mlp_free(h_);
        h_ = nullptr;
        b200fc_detail::check(b200fc_mlp_create(w_gate, w_up, w_down, K, N, 0, 1, &h_, nullptr));
        m_K = K; m_N = N;
    }
    void run(uint8_t* pA, int strideA, int M, ov::bfloat16* dstC, int strideC) {
        if (!h_) throw std::runtime_error("MLP::run before setup");
        b200fc_detail::check(b200fc_mlp_run_host(h_, pA, strideA, M, dstC, strideC, nullptr));
    }
    int m_K = 0, m_N = 0;

private:
    b200fc_mlp_t* h_ = nullptr;
};
}  // namespace AMX_MLP
