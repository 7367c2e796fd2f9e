// Matrix x vector: c[M] = A[M, K] * b[K].
//
// Replaces amx_kernel::MatmulVector::operator() (include/kernels_amx.hpp:959-1042; the q·K^T-style product with
// K <= 6 AMX tiles) and the AVX-512 GemAvB (kernels_amx.hpp:1529-1618).  The reference limits K to 32..192 (bf16) /
// 64..384 (int8) because the vector must fit six tile registers; here any K works.  The op is an HBM-bound stream of
// A: one warp per row, 16-byte loads along K when the row base allows, warp-shuffle reduction.  bf16 products are
// accumulated in fp32, int8 products exactly in int32 (dp4a).
#include "common.cuh"

namespace b200fc {

namespace {

__device__ __forceinline__ float bf16_lo(unsigned v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(unsigned v) { return __uint_as_float(v & 0xffff0000u); }

__global__ void matvec_bf16_kernel(const unsigned char* __restrict__ A, long long lda, int M, int K,
                                   const unsigned short* __restrict__ b, float* __restrict__ c) {
    const int lane = threadIdx.x & 31;
    const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    const bool b_vec = ((uintptr_t)b & 15) == 0;
    for (int m = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; m < M; m += warps_per_grid) {
        const unsigned char* row = A + (long long)m * lda;
        float s = 0.0f;
        int k0 = 0;
        if ((((uintptr_t)row) & 15) == 0 && b_vec) {
            const int nvec = K / 8;
            for (int v = lane; v < nvec; v += 32) {
                uint4 a = *(const uint4*)(row + (long long)v * 16);
                uint4 x = __ldg((const uint4*)b + v);
                s = fmaf(bf16_lo(a.x), bf16_lo(x.x), s); s = fmaf(bf16_hi(a.x), bf16_hi(x.x), s);
                s = fmaf(bf16_lo(a.y), bf16_lo(x.y), s); s = fmaf(bf16_hi(a.y), bf16_hi(x.y), s);
                s = fmaf(bf16_lo(a.z), bf16_lo(x.z), s); s = fmaf(bf16_hi(a.z), bf16_hi(x.z), s);
                s = fmaf(bf16_lo(a.w), bf16_lo(x.w), s); s = fmaf(bf16_hi(a.w), bf16_hi(x.w), s);
            }
            k0 = nvec * 8;
        }
        for (int k = k0 + lane; k < K; k += 32)
            s = fmaf(bf16_lo(((const unsigned short*)row)[k]), bf16_lo(b[k]), s);
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) c[m] = s;
    }
}

__global__ void matvec_s8_kernel(const unsigned char* __restrict__ A, long long lda, int M, int K,
                                 const signed char* __restrict__ b, int* __restrict__ c) {
    const int lane = threadIdx.x & 31;
    const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    const bool b_vec = ((uintptr_t)b & 15) == 0;
    for (int m = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; m < M; m += warps_per_grid) {
        const unsigned char* row = A + (long long)m * lda;
        int s = 0;
        int k0 = 0;
        if ((((uintptr_t)row) & 15) == 0 && b_vec) {
            const int nvec = K / 16;
            for (int v = lane; v < nvec; v += 32) {
                int4 a = *(const int4*)(row + (long long)v * 16);
                int4 x = __ldg((const int4*)b + v);
                s = __dp4a(a.x, x.x, s); s = __dp4a(a.y, x.y, s);
                s = __dp4a(a.z, x.z, s); s = __dp4a(a.w, x.w, s);
            }
            k0 = nvec * 16;
        }
        for (int k = k0 + lane; k < K; k += 32) s += (int)((const signed char*)row)[k] * (int)b[k];
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) c[m] = s;
    }
}

}  // namespace

int launch_matvec(const void* A, int dtype, int M, int K, int64_t lda, const void* b, void* c, cudaStream_t s) {
    if (M <= 0) return B200FC_OK;
    const int block = 256, warps_per_block = block / 32;
    long long blocks = (M + warps_per_block - 1) / warps_per_block;
    if (blocks > 148 * 8) blocks = 148 * 8;  // whole waves of 8 resident CTAs per SM
    if (dtype == B200FC_BF16)
        matvec_bf16_kernel<<<(unsigned)blocks, block, 0, s>>>((const unsigned char*)A, lda, M, K, (const unsigned short*)b, (float*)c);
    else if (dtype == B200FC_S8)
        matvec_s8_kernel<<<(unsigned)blocks, block, 0, s>>>((const unsigned char*)A, lda, M, K, (const signed char*)b, (int*)c);
    else { set_error("matvec: dtype must be bf16 or s8"); return B200FC_ERR_INVALID; }
    count_launch();
    B200FC_CUDA(cudaGetLastError());
    return B200FC_OK;
}

}  // namespace b200fc
