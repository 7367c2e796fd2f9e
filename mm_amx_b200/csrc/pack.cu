// Weight packing and small data-movement kernels.
//
// Replaces amx_kernel::repackB_1x2 (include/kernels_amx.hpp:761-816) and, for compressed weights, get_min_max +
// bf16_to_i8_tensor (kernels_amx.hpp:465-488, 508-523).  The AMX code packs B into 16x64-byte VNNI tiles; the
// tcgen05 tensor core instead wants K-major rows that a 128-byte-swizzled TMA box can drop into shared memory, so
// the packed form here is a zero-padded row-major [N_pad, K_pad] matrix (K contiguous).  All kernels are HBM-bound
// byte movers: coalesced reads along the source's contiguous dimension, a shared-memory tile transpose when the
// source is [K, N], coalesced writes.
#include "common.cuh"

namespace b200fc {

namespace {

constexpr int TILE = 64;

enum PackMode { PLAIN16 = 0, PLAIN8 = 1, QUANT8 = 2 };

template <int MODE> struct SrcT { using type = unsigned short; };
template <> struct SrcT<PLAIN8> { using type = unsigned char; };
template <int MODE> struct DstT { using type = unsigned char; };
template <> struct DstT<PLAIN16> { using type = unsigned short; };

template <int MODE>
__device__ __forceinline__ typename DstT<MODE>::type convert(typename SrcT<MODE>::type v, float qscale) {
    if constexpr (MODE == QUANT8) {
        // bf16 -> fp32 -> * quant scale -> round to nearest even -> saturate (bf16_to_i8_tensor, :508-523)
        float f = __uint_as_float((unsigned)v << 16) * qscale;
        return (unsigned char)(signed char)f32_to_s8(f);
    } else {
        return v;
    }
}

// dst[n, k] = src[k, n] (transposeB = 0) or src[n, k] (transposeB = 1); zero outside [N) x [K).
// grid: (K_pad / TILE, N_pad / TILE), block: (TILE, 4)
template <int MODE>
__global__ void pack_kernel(const void* __restrict__ src_, long long lds, int K, int N, int transposeB,
                            void* __restrict__ dst_, int K_pad, const float* __restrict__ absmax, int flip) {
    using S = typename SrcT<MODE>::type;
    using D = typename DstT<MODE>::type;
    __shared__ S tile[TILE][TILE + 2];
    const int k0 = blockIdx.x * TILE, n0 = blockIdx.y * TILE;
    const int tx = threadIdx.x, ty = threadIdx.y;
    float qscale = 1.0f;
    if constexpr (MODE == QUANT8) qscale = __fdiv_rn(127.0f, *absmax);
    const char* src = (const char*)src_;
    D* dst = (D*)dst_;
    // compressed weights are stored offset-binary (value + 128, padding included): see gemv.cu
    const D fl = (D)(flip ? 0x80 : 0);
    if (transposeB) {
        for (int r = ty; r < TILE; r += blockDim.y) {
            int n = n0 + r, k = k0 + tx;
            S v = 0;
            if (n < N && k < K) v = *(const S*)(src + (long long)n * lds + (long long)k * sizeof(S));
            dst[(long long)n * K_pad + k] = convert<MODE>(v, qscale) ^ fl;
        }
    } else {
        for (int r = ty; r < TILE; r += blockDim.y) {
            int k = k0 + r, n = n0 + tx;
            S v = 0;
            if (n < N && k < K) v = *(const S*)(src + (long long)k * lds + (long long)n * sizeof(S));
            tile[r][tx] = v;
        }
        __syncthreads();
        for (int r = ty; r < TILE; r += blockDim.y) {
            int n = n0 + r, k = k0 + tx;
            dst[(long long)n * K_pad + k] = convert<MODE>(tile[tx][r], qscale) ^ fl;
        }
    }
}

// Fused-MLP weight: packed row 32q + i is gate row 16q + i for i < 16 and up row 16q + i - 16 otherwise, so one
// accumulator tile holds gate and up of the same 16 channels (the interleave of MLP::setup,
// tests/amx-mlp.cpp:758-765).  gate / up are [rows, K] bf16 with leading dimension lds; 8 elements per thread.
__global__ void pack_gate_up_kernel(const unsigned short* __restrict__ gate, const unsigned short* __restrict__ up,
                                    long long lds_elems, int K, int rows, unsigned short* __restrict__ dst, int K_pad,
                                    int N_pad) {
    const int per_row = K_pad / 8;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)N_pad * per_row) return;
    const int r = (int)(i / per_row), k = (int)(i % per_row) * 8;
    const int q = r >> 5, j = r & 31;
    const int src_row = 16 * q + (j & 15);
    const unsigned short* src = (j < 16 ? gate : up) + (long long)src_row * lds_elems;
    __align__(16) unsigned short o[8];
#pragma unroll
    for (int e = 0; e < 8; e++) o[e] = (src_row < rows && k + e < K) ? src[k + e] : (unsigned short)0;
    *(int4*)(dst + (long long)r * K_pad + k) = *(int4*)o;
}

// absmax over a bf16 matrix (get_min_max, :465-488, followed by max(|min|, |max|), :1371).  Non-negative floats
// order like their bit patterns, so the reduction ends in an integer atomicMax.
__global__ void absmax_kernel(const void* __restrict__ src_, long long lds, int rows, int cols,
                              unsigned* __restrict__ out_bits) {
    const char* src = (const char*)src_;
    float m = 0.0f;
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const unsigned short* row = (const unsigned short*)(src + (long long)r * lds);
        for (int c = threadIdx.x; c < cols; c += blockDim.x)
            m = fmaxf(m, fabsf(__uint_as_float((unsigned)row[c] << 16)));
    }
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) atomicMax(out_bits, __float_as_uint(m));
}

// compressed weights (offset-binary int8) [N_pad, K_pad] -> bf16 [N_pad, dst_K_pad] (exact: |v| <= 128 fits the
// 8-bit significand of bf16); i8_to_bf16_Kx32, include/kernels_amx.hpp:490-506.  16 elements per thread.
__global__ void dequant_bf16_kernel(const signed char* __restrict__ src, int K_pad, long long total16,
                                    unsigned short* __restrict__ dst, int dst_K_pad) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total16) return;
    int per_row = K_pad / 16;
    long long n = i / per_row;
    int k = (int)(i % per_row) * 16;
    int4 v = *(const int4*)(src + n * K_pad + k);
    const unsigned char* b = (const unsigned char*)&v;
    __align__(16) unsigned short o[16];
#pragma unroll
    for (int j = 0; j < 16; j++) o[j] = f32_to_bf16_bits((float)((int)b[j] - 128));
    int4* d = (int4*)(dst + n * dst_K_pad + k);
    d[0] = *(int4*)&o[0];
    d[1] = *(int4*)&o[8];
}

// ---- 4-bit group-quantised weights -----------------------------------------------------------------------------------
// Stored form: the byte matrix [N_pad, K_pad / 2]; a value v in [-7, 7] is the nibble v + 8.  Every 128-byte piece of a
// row (256 values, one stage of the decode kernel) holds two groups of 128 K; its eight 16-byte units alternate between
// them (unit u holds values [32 * (u >> 1), +32) of group u & 1), so that the four lanes whose fragments one MMA of the
// decode kernel combines (units 2t + h, t = 0..3) stay inside ONE group and the group's scale can be applied to the
// MMA's sum.  Inside a 32-bit word the eight values k .. k + 7 sit at nibble positions 0, 4, 1, 5, 2, 6, 3, 7: masking
// with 0x000f000f / 0x00f000f0 (and once more after a shift by 8) then yields K-neighbours as the two halves of a
// 16-bit pair, the order the MMA fragment wants.
__device__ __forceinline__ int nibble_pos(int e) { return (e >> 1) + 4 * (e & 1); }
// first K of the eight values held by the word at byte offset `off` of a packed row
__device__ __forceinline__ int word_k0(int off) {
    const int ks = off >> 7, u = (off >> 4) & 7, wq = (off >> 2) & 3;
    return ks * 256 + (u & 1) * 128 + (u >> 1) * 32 + wq * 8;
}

// One warp quantises one group (128 consecutive K of one row) of the zero-padded bf16 matrix `wide` [N_pad, K_pad]:
// absmax -> quant scale 7 / absmax (fp32 division; 0 for an all-zero group) -> round to nearest even, and stores the
// dequant scale absmax / 7 where the decode kernel's stage finds it.
__global__ void __launch_bounds__(256) quant4_kernel(const unsigned short* __restrict__ wide, int K_pad, long long groups,
                                                     unsigned* __restrict__ dst, float* __restrict__ scale_grp) {
    const long long gi = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (gi >= groups) return;
    const int lane = threadIdx.x & 31;
    const int gpr = K_pad / 128;
    const long long n = gi / gpr;
    const int j = (int)(gi % gpr);
    const uint2 raw = *(const uint2*)(wide + n * K_pad + j * 128 + lane * 4);
    const float f[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16),
                        __uint_as_float(raw.y & 0xffff0000u)};
    float m = fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float qs = m > 0.0f ? __fdiv_rn(7.0f, m) : 0.0f;
    unsigned word = 0;
#pragma unroll
    for (int e = 0; e < 4; e++) {
        int v = f32_to_s8(__fmul_rn(f[e], qs));
        v = v > 7 ? 7 : (v < -7 ? -7 : v);
        word |= (unsigned)((v + 8) & 15) << (4 * nibble_pos(4 * (lane & 1) + e));
    }
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    const int ks = j >> 1, gh = j & 1;
    if (!(lane & 1)) {
        const int wi = lane >> 1, b = wi >> 2, wq = wi & 3;
        dst[(n * (K_pad / 2) + ks * 128 + (b * 2 + gh) * 16 + wq * 4) >> 2] = word;
    }
    if (lane == 0) scale_grp[((((n >> 7) * (K_pad / 256)) + ks) * 2 + gh) * 128 + (n & 127)] = __fdiv_rn(m, 7.0f);
}

__device__ __forceinline__ float scale4_at(const float* scale_grp, int K_pad, long long n, int k) {
    return scale_grp[((((n >> 7) * (K_pad / 256)) + (k >> 8)) * 2 + ((k >> 7) & 1)) * 128 + (n & 127)];
}

// packed rows [row0, row0 + rows) -> one int8 per value (dst_s8, rows x K) or value * group scale rounded to bf16
// (dst_bf16, rows x dst_K_pad, zero padded like the source); one 32-bit word (8 values) per thread
__global__ void unpack4_kernel(const unsigned* __restrict__ src, int K_pad, const float* __restrict__ scale_grp, int row0,
                               long long words, signed char* __restrict__ dst_s8, long long ldd, int N, int K,
                               unsigned short* __restrict__ dst_bf16, int dst_K_pad) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= words) return;
    const int wpr = K_pad / 8;
    const long long r = i / wpr, n = row0 + r;
    const int off = (int)(i % wpr) * 4;
    const unsigned word = src[(n * (K_pad / 2) + off) >> 2];
    const int k0 = word_k0(off);
    if (dst_s8) {
        if (n >= N) return;
#pragma unroll
        for (int e = 0; e < 8; e++)
            if (k0 + e < K) dst_s8[n * ldd + k0 + e] = (signed char)((int)((word >> (4 * nibble_pos(e))) & 15) - 8);
    } else {
        const float sc = scale4_at(scale_grp, K_pad, n, k0);
        __align__(16) unsigned short o[8];
#pragma unroll
        for (int e = 0; e < 8; e++) o[e] = f32_to_bf16_bits((float)((int)((word >> (4 * nibble_pos(e))) & 15) - 8) * sc);
        *(int4*)(dst_bf16 + r * dst_K_pad + k0) = *(int4*)o;
    }
}

// row-wise copy with zero fill of [row_bytes, dst_row_bytes): re-strides an activation matrix whose leading
// dimension or base address does not meet the 16-byte rules of a TMA descriptor.
__global__ void copy2d_kernel(const char* __restrict__ src, long long lds, char* __restrict__ dst, long long ldd,
                              int rows, int row_bytes, int dst_row_bytes) {
    for (int r = blockIdx.x; r < rows; r += gridDim.x)
        for (int c = threadIdx.x; c < dst_row_bytes; c += blockDim.x)
            dst[(long long)r * ldd + c] = c < row_bytes ? src[(long long)r * lds + c] : (char)0;
}

// dst[r, c] = src[r, c] ^ 0x80: offset-binary <-> two's complement, row-wise with independent strides
__global__ void flip_copy2d_kernel(const unsigned char* __restrict__ src, long long lds, unsigned char* __restrict__ dst,
                                   long long ldd, int rows, int cols) {
    for (int r = blockIdx.x; r < rows; r += gridDim.x)
        for (int c = threadIdx.x; c < cols; c += blockDim.x) dst[(long long)r * ldd + c] = src[(long long)r * lds + c] ^ 0x80;
}

__global__ void add_round_bf16_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                      unsigned short* __restrict__ out, long long n) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = f32_to_bf16_bits(b ? a[i] + b[i] : a[i]);
}

// RMS normalisation of one row per block, the LlamaRMSNorm the reference's benchmark script puts in front of every MLP
// (torch-ext/test.py:161-176): fp32 arithmetic, y = x * rsqrt(mean(x^2) + eps), rounded to bf16; an optional bf16
// weight vector multiplies the rounded value (the transformers form), rounded again.
__global__ void __launch_bounds__(256) rmsnorm_kernel(const unsigned short* __restrict__ x, long long ldx, int K,
                                                      const unsigned short* __restrict__ weight, float eps,
                                                      unsigned short* __restrict__ out, long long ldo) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const unsigned short* row = (const unsigned short*)((const char*)x + (long long)blockIdx.x * ldx);
    unsigned short* orow = (unsigned short*)((char*)out + (long long)blockIdx.x * ldo);
    float ss = 0.0f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
        const float v = __uint_as_float((unsigned)row[k] << 16);
        ss = fmaf(v, v, ss);
    }
    __shared__ float red[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += red[i];      // same order in every thread
    const float r = rsqrtf(tot / (float)K + eps);
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
        unsigned short y = f32_to_bf16_bits(__uint_as_float((unsigned)row[k] << 16) * r);
        if (weight) y = f32_to_bf16_bits(__uint_as_float((unsigned)y << 16) * __uint_as_float((unsigned)weight[k] << 16));
        orow[k] = y;
    }
}

__global__ void fill_kernel(int4* __restrict__ p, long long n16, int v) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n16; i += stride) p[i] = make_int4(v, v, v, v);
}

}  // namespace

int launch_pack(const void* B, int dtypeB, int K, int N, int64_t ldb, int transposeB, Weight& w, bool offset_binary,
                cudaStream_t s) {
    dim3 grid((w.K_pad + TILE - 1) / TILE, w.N_pad / TILE), block(TILE, 4);
    if (dtypeB == B200FC_BF16)
        pack_kernel<PLAIN16><<<grid, block, 0, s>>>(B, ldb, K, N, transposeB, w.data, w.K_pad, nullptr, 0);
    else
        pack_kernel<PLAIN8><<<grid, block, 0, s>>>(B, ldb, K, N, transposeB, w.data, w.K_pad, nullptr, offset_binary ? 1 : 0);
    count_launch();
    B200FC_CUDA(cudaGetLastError());
    return B200FC_OK;
}

int launch_pack_gate_up(const void* gate, const void* up, int64_t ld_bytes, int K, int rows, Weight& w, cudaStream_t s) {
    long long total = (long long)w.N_pad * (w.K_pad / 8);
    pack_gate_up_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>((const unsigned short*)gate, (const unsigned short*)up,
                                                                     ld_bytes / 2, K, rows, (unsigned short*)w.data,
                                                                     w.K_pad, w.N_pad);
    count_launch();
    B200FC_CUDA(cudaGetLastError());
    return B200FC_OK;
}

int launch_absmax(const void* B, int rows, int cols, int64_t ldb, float* absmax_dev, cudaStream_t s) {
    B200FC_CUDA(cudaMemsetAsync(absmax_dev, 0, sizeof(float), s));
    int grid = rows < 1184 ? rows : 1184;
    absmax_kernel<<<grid, 256, 0, s>>>(B, ldb, rows, cols, (unsigned*)absmax_dev);
    count_launch();
    B200FC_CUDA(cudaGetLastError());
    return B200FC_OK;
}

int launch_quant_pack(const void* B, int K, int N, int64_t ldb, int transposeB, Weight& w, float* absmax_dev,
                      cudaStream_t s) {
    dim3 grid((w.K_pad + TILE - 1) / TILE, w.N_pad / TILE), block(TILE, 4);
    pack_kernel<QUANT8><<<grid, block, 0, s>>>(B, ldb, K, N, transposeB, w.data, w.K_pad, absmax_dev, 1);
    count_launch();
    B200FC_CUDA(cudaGetLastError());
    return B200FC_OK;
}

int launch_quant4(const void* wide_bf16, Weight& w, cudaStream_t s) {
    const long long groups = (long long)w.N_pad * (w.K_pad / 128);
    quant4_kernel<<<(unsigned)((groups * 32 + 255) / 256), 256, 0, s>>>((const unsigned short*)wide_bf16, w.K_pad, groups,
                                                                        (unsigned*)w.data, w.scale_grp);
    count_launch();
    B200FC_CUDA(cudaGetLastError());
    return B200FC_OK;
}

int launch_unpack4(const Weight& w, void* dst_s8, int64_t ldd, cudaStream_t s) {
    const long long words = (long long)w.N_pad * (w.K_pad / 8);
    unpack4_kernel<<<(unsigned)((words + 255) / 256), 256, 0, s>>>((const unsigned*)w.data, w.K_pad, w.scale_grp, 0, words,
                                                                   (signed char*)dst_s8, ldd, w.N, w.K, nullptr, 0);
    count_launch();
    B200FC_CUDA(cudaGetLastError());
    return B200FC_OK;
}

int launch_dequant_bf16(const Weight& w, int row0, int rows, void* dst, int dst_K_pad, cudaStream_t s) {
    // rows [row0, row0 + rows) of the packed matrix -> dst rows [0, rows)
    if (w.dtype == B200FC_S4) {
        const long long words = (long long)rows * (w.K_pad / 8);
        unpack4_kernel<<<(unsigned)((words + 255) / 256), 256, 0, s>>>((const unsigned*)w.data, w.K_pad, w.scale_grp, row0,
                                                                       words, nullptr, 0, w.N, w.K, (unsigned short*)dst,
                                                                       dst_K_pad);
        count_launch();
        B200FC_CUDA(cudaGetLastError());
        return B200FC_OK;
    }
    long long total16 = (long long)rows * (w.K_pad / 16);
    int block = 256;
    long long grid = (total16 + block - 1) / block;
    dequant_bf16_kernel<<<(unsigned)grid, block, 0, s>>>((const signed char*)w.data + (size_t)row0 * w.K_pad, w.K_pad,
                                                         total16, (unsigned short*)dst, dst_K_pad);
    count_launch();
    B200FC_CUDA(cudaGetLastError());
    return B200FC_OK;
}

int launch_copy2d(const void* src, int64_t lds, void* dst, int64_t ldd, int rows, int row_bytes, int dst_row_bytes,
                  cudaStream_t s) {
    int grid = rows < 2368 ? rows : 2368;
    copy2d_kernel<<<grid, 256, 0, s>>>((const char*)src, lds, (char*)dst, ldd, rows, row_bytes, dst_row_bytes);
    count_launch();
    B200FC_CUDA(cudaGetLastError());
    return B200FC_OK;
}

int launch_flip_copy2d(const void* src, int64_t lds, void* dst, int64_t ldd, int rows, int cols, cudaStream_t s) {
    int grid = rows < 2368 ? rows : 2368;
    flip_copy2d_kernel<<<grid, 256, 0, s>>>((const unsigned char*)src, lds, (unsigned char*)dst, ldd, rows, cols);
    count_launch();
    B200FC_CUDA(cudaGetLastError());
    return B200FC_OK;
}

int launch_add_round_bf16(const float* a, const float* b, void* out, int64_t n, cudaStream_t s) {
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks < 1) blocks = 1;
    add_round_bf16_kernel<<<(unsigned)blocks, 256, 0, s>>>(a, b, (unsigned short*)out, n);
    count_launch();
    B200FC_CUDA(cudaGetLastError());
    return B200FC_OK;
}

int launch_rmsnorm(const void* x, int64_t ldx, int M, int K, const void* weight, float eps, void* out, int64_t ldo,
                   cudaStream_t s) {
    if (M <= 0) return B200FC_OK;
    rmsnorm_kernel<<<M, 256, 0, s>>>((const unsigned short*)x, ldx, K, (const unsigned short*)weight, eps,
                                     (unsigned short*)out, ldo);
    count_launch();
    B200FC_CUDA(cudaGetLastError());
    return B200FC_OK;
}

int launch_fill(void* p, size_t bytes, cudaStream_t s) {
    fill_kernel<<<148 * 8, 256, 0, s>>>((int4*)p, (long long)(bytes / 16), 0);
    count_launch();
    B200FC_CUDA(cudaGetLastError());
    return B200FC_OK;
}

}  // namespace b200fc
