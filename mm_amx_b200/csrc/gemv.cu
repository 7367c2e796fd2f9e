// Decode-shaped fully-connected layer (M <= 16 rows of bf16 activations) — an HBM-bound weight stream.
//
// Replaces the M <= 16 branches of amx_kernel::Matmul (include/kernels_amx.hpp:1216-1253), of the compressed-weight
// specialisation Matmul<bf16,int8_t,float> (kernels_amx.hpp:1381-1441) and its stand-alone development version
// matmul16m_Wint8B (weight_compression/fc16m.cpp:451-502), plus the M <= 16 case of the fused MLP
// (tests/amx-mlp.cpp:707-737, 648-704).
//
// How the bytes move
//   The packed weights are [N_pad, K_pad] with K contiguous.  A warp owns 32 output channels (two 16-row blocks).
//   Thread (g = lane / 4, t = lane % 4) streams rows g and g + 8 of each block with 16-byte
//   ld.global.nc.L1::no_allocate loads: per 64-byte K block it takes bytes [16t, 16t + 16) of its rows, so four
//   neighbouring lanes cover one 64-byte segment.  Loads are issued a pipeline stage (2 K blocks, 8 loads per thread)
//   ahead of their use and two stages stay in flight, so a warp always has 8 KB outstanding.
//   The loaded registers ARE the A fragments of mma.sync.m16n8k16 (weights as the 16-row operand, the <= 16
//   activation rows as the 8-column operand): K is permuted identically for both operands, which is free because
//   a dot product does not care about the order of its terms per MMA slot.  Compressed (int8) weights are widened in
//   registers right before the MMA — the "dequantise next to the consumer" idea of the reference's ping-pong
//   buffer, without the buffer.  They are stored offset-binary (v + 128) so that one byte permute builds the fp16
//   number 1024 + v + 128 and one subtraction leaves v: one instruction per weight.  fp16 (not bf16) because only
//   its 10-bit mantissa holds all 8 bits; the activations are therefore converted to fp16 per staged chunk, after
//   an exact power-of-two scaling per row that keeps them inside the fp16 range.  A SIMT dot product cannot keep up with HBM3e at M = 16 (16 FMAs per weight byte), the
//   tensor-core path can; at M = 1 the seven unused columns cost nothing.
//   Activations are staged in shared memory in chunks of 1024 K elements (padded rows, conflict-free 16-byte reads).
//   Split-K: S CTAs of a thread-block cluster share a row range and split K; partial sums meet in distributed shared
//   memory and are added in rank order (deterministic), then the post-ops run and C is stored.
#include <cooperative_groups.h>
#include <cuda_fp16.h>
#include <cstdlib>
#include "common.cuh"

namespace cg = cooperative_groups;

namespace b200fc {

namespace {

constexpr int WARPS = 4;
constexpr int ROWS_PER_WARP = 32;
constexpr int ROWS_PER_CTA = WARPS * ROWS_PER_WARP;  // 128
constexpr int KB_BYTES = 64;                          // one K block = 64 bytes of a weight row
constexpr int KB_PER_ITER = 2;                        // K blocks per pipeline stage
constexpr int CHUNK_K = 1024;                         // activation elements staged per chunk

struct GemvParams {
    const unsigned char* W;  // packed weights
    long long ldw;           // bytes
    int N_pad;
    const unsigned char* X;  // activations [M, K] bf16
    long long ldx;           // bytes
    int M, K;
    int n_kb;                // K blocks in a packed row (K_pad bytes / 64)
    int n0, n1;
    int splits;
    Epilogue ep;
};

__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_f16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                        unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Two compressed weights (bytes `sel` of w, stored offset-binary: u = v + 128) -> f16x2 holding v exactly, in two
// instructions: 0x6400 | u is the fp16 number 1024 + u (u fits the 10-bit mantissa), minus 1152 leaves v.
__device__ __forceinline__ unsigned u8x2_to_f16x2(unsigned w, unsigned sel) {
    unsigned p = __byte_perm(w, 0x64646464u, sel);
    const __half2 off = __floats2half2_rn(1152.0f, 1152.0f);
    __half2 r = __hsub2(*(__half2*)&p, off);
    return *(unsigned*)&r;
}

template <bool W8, int NT>
__global__ void __launch_bounds__(WARPS * 32, 4) gemv_kernel(const GemvParams p) {
    constexpr int KB_ELEMS = W8 ? 64 : 32;                  // K elements per K block
    constexpr int MP = 8 * NT;                              // padded activation rows
    constexpr int XROW = CHUNK_K * 2 + (W8 ? 16 : 64);      // bytes per staged activation row (bank-conflict free)
    constexpr int ITERS_PER_CHUNK = CHUNK_K / (KB_ELEMS * KB_PER_ITER);
    constexpr int MMA_PER_LOAD = W8 ? 4 : 2;

    extern __shared__ __align__(16) unsigned char smem[];   // MP * XROW bytes; later reused for the partial tile

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    cg::cluster_group cluster = cg::this_cluster();
    const int S = p.splits;
    const int rank = S > 1 ? (int)cluster.block_rank() : 0;

    // K range of this split, in iterations of KB_PER_ITER K blocks
    const int iters_total = (p.n_kb + KB_PER_ITER - 1) / KB_PER_ITER;
    const int it_begin = (int)((long long)iters_total * rank / S);
    const int it_end = (int)((long long)iters_total * (rank + 1) / S);

    const int cta_row0 = p.n0 + blockIdx.x * ROWS_PER_CTA;
    const int warp_row0 = cta_row0 + warp * ROWS_PER_WARP;

    // the four weight rows this thread streams (clamped into the padded matrix; clamped rows are never stored)
    const unsigned char* wrow[2][2];
#pragma unroll
    for (int rb = 0; rb < 2; rb++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            int r = warp_row0 + rb * 16 + h * 8 + g;
            r = r < p.N_pad ? r : p.N_pad - 1;
            wrow[rb][h] = p.W + (long long)r * p.ldw + 16 * t;
        }

    float acc[2][NT][4];
#pragma unroll
    for (int rb = 0; rb < 2; rb++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[rb][nt][i] = 0.0f;

    const bool x_vec = (((uintptr_t)p.X & 15) == 0) && ((p.ldx & 15) == 0);
    int cur_e[NT][2];  // compressed weights: power-of-two scale of the staged activations, per token of this thread
#pragma unroll
    for (int nt = 0; nt < NT; nt++) cur_e[nt][0] = cur_e[nt][1] = 0;

    // One pipeline stage = KB_PER_ITER K blocks of the warp's four rows (8 x 16-byte loads per thread).  Two stages
    // are kept in flight: the loads of stage i+1 are issued before stage i is multiplied.
    uint4 wbuf[2][2][2][KB_PER_ITER];
    auto issue = [&](int buf, int it) {
        const int kb0 = it * KB_PER_ITER;
#pragma unroll
        for (int j = 0; j < KB_PER_ITER; j++) {
            const bool in = it < it_end && kb0 + j < p.n_kb;
#pragma unroll
            for (int rb = 0; rb < 2; rb++)
#pragma unroll
                for (int h = 0; h < 2; h++)
                    wbuf[buf][rb][h][j] = in ? ld_stream(wrow[rb][h] + (long long)(kb0 + j) * KB_BYTES) : make_uint4(0, 0, 0, 0);
        }
    };
    // one 16-byte unit (8 bf16) of activation row `row` at K element k; zero beyond M rows / K columns (the padded
    // weights are zero there, the activations must not be garbage)
    auto load_x_unit = [&](int row, int k) -> uint4 {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < p.M && k < p.K) {
            const unsigned char* src = p.X + (long long)row * p.ldx + (long long)k * 2;
            if (x_vec && k + 8 <= p.K) {
                v = *(const uint4*)src;
            } else {
                unsigned short e[8];
#pragma unroll
                for (int q = 0; q < 8; q++) e[q] = (k + q < p.K) ? ((const unsigned short*)src)[q] : (unsigned short)0;
                v.x = e[0] | ((unsigned)e[1] << 16); v.y = e[2] | ((unsigned)e[3] << 16);
                v.z = e[4] | ((unsigned)e[5] << 16); v.w = e[6] | ((unsigned)e[7] << 16);
            }
        }
        return v;
    };
    // Stages the activation chunk that starts at iteration `it`: CHUNK_K elements of MP rows, one 16-byte unit per
    // thread and row.  bf16 weights: the bf16 activations are copied as they are.  Compressed weights: the tensor
    // core multiplies fp16 x fp16 there, so each row of the chunk is scaled by a power of two that puts its largest
    // magnitude at 2^13 (exact; fp16 keeps the 8-bit significand of bf16) and converted to fp16; the accumulators
    // carry the scale (cur_e) and are rescaled when it changes.
    auto stage_x = [&](int it) {
        const int chunk_k0 = it * KB_PER_ITER * KB_ELEMS;
        const int k = chunk_k0 + threadIdx.x * 8;
        const bool need = k < it_end * KB_PER_ITER * KB_ELEMS;  // nothing beyond this split's K range is read
        __syncthreads();  // everyone is done with the previous chunk
        if constexpr (W8) {
            unsigned* smax = (unsigned*)(smem + MP * XROW);       // [MP][WARPS] largest |bits| seen per row and warp
            int* sexp = (int*)(smem + MP * XROW + MP * WARPS * 4); // [MP] scale exponent of the row
#pragma unroll 1
            for (int row = 0; row < MP; row++) {
                unsigned m = 0;
                if (need) {
                    const uint4 v = load_x_unit(row, k);
                    const unsigned w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int q = 0; q < 4; q++) m = max(m, max(w4[q] & 0x7fffu, (w4[q] >> 16) & 0x7fffu));
                }
                m = __reduce_max_sync(0xffffffffu, m);
                if (lane == 0) smax[row * WARPS + warp] = m;
            }
            __syncthreads();
#pragma unroll 1
            for (int row = 0; row < MP; row++) {
                unsigned m = 0;
#pragma unroll
                for (int q = 0; q < WARPS; q++) m = max(m, smax[row * WARPS + q]);
                int field = (int)(m >> 7);                 // biased exponent of the largest magnitude (bf16 layout)
                field = field < 1 ? 1 : field;
                int e = field - 127 - 13;
                e = e < -126 ? -126 : e;
                if (threadIdx.x == 0) sexp[row] = e;
                if (need) {
                    const float sc = __int_as_float((127 - e) << 23);  // 2^-e
                    const uint4 v = load_x_unit(row, k);
                    const unsigned w4[4] = {v.x, v.y, v.z, v.w};
                    unsigned o[4];
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        __half2 h = __floats2half2_rn(__uint_as_float(w4[q] << 16) * sc,
                                                      __uint_as_float(w4[q] & 0xffff0000u) * sc);
                        o[q] = *(unsigned*)&h;
                    }
                    *(uint4*)(smem + row * XROW + threadIdx.x * 16) = make_uint4(o[0], o[1], o[2], o[3]);
                }
            }
        } else {
#pragma unroll 1
            for (int row = 0; row < MP; row++)
                if (need) *(uint4*)(smem + row * XROW + threadIdx.x * 16) = load_x_unit(row, k);
        }
        __syncthreads();
        if constexpr (W8) {
            // bring the running sums to the new chunk's scale: acc holds sum * 2^-cur_e
            const int* sexp = (const int*)(smem + MP * XROW + MP * WARPS * 4);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int e0 = sexp[nt * 8 + 2 * t], e1 = sexp[nt * 8 + 2 * t + 1];
                if (cur_e[nt][0] != e0 || cur_e[nt][1] != e1) {
#pragma unroll
                    for (int rb = 0; rb < 2; rb++) {
                        acc[rb][nt][0] = scalbnf(acc[rb][nt][0], cur_e[nt][0] - e0);
                        acc[rb][nt][2] = scalbnf(acc[rb][nt][2], cur_e[nt][0] - e0);
                        acc[rb][nt][1] = scalbnf(acc[rb][nt][1], cur_e[nt][1] - e1);
                        acc[rb][nt][3] = scalbnf(acc[rb][nt][3], cur_e[nt][1] - e1);
                    }
                    cur_e[nt][0] = e0; cur_e[nt][1] = e1;
                }
            }
        }
    };
    auto multiply = [&](int buf, int it_in_chunk) {
#pragma unroll
        for (int j = 0; j < KB_PER_ITER; j++) {
            // activation fragments of this K block: per row, the bytes matching this thread's weight bytes
            const int xoff = (it_in_chunk * KB_PER_ITER + j) * KB_ELEMS * 2 + t * (W8 ? 32 : 16);
            unsigned xb[NT][W8 ? 8 : 4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const unsigned char* xs = smem + (nt * 8 + g) * XROW + xoff;
                uint4 a = *(const uint4*)xs;
                xb[nt][0] = a.x; xb[nt][1] = a.y; xb[nt][2] = a.z; xb[nt][3] = a.w;
                if constexpr (W8) {
                    uint4 b = *(const uint4*)(xs + 16);
                    xb[nt][4] = b.x; xb[nt][5] = b.y; xb[nt][6] = b.z; xb[nt][7] = b.w;
                }
            }
#pragma unroll
            for (int rb = 0; rb < 2; rb++) {
                const uint4 va = wbuf[buf][rb][0][j], vb = wbuf[buf][rb][1][j];
                const unsigned wa[4] = {va.x, va.y, va.z, va.w};  // row g
                const unsigned wb[4] = {vb.x, vb.y, vb.z, vb.w};  // row g + 8
#pragma unroll
                for (int q = 0; q < MMA_PER_LOAD; q++) {
                    unsigned a0, a1, a2, a3;
                    if constexpr (W8) {
                        a0 = u8x2_to_f16x2(wa[q], 0x4140); a2 = u8x2_to_f16x2(wa[q], 0x4342);
                        a1 = u8x2_to_f16x2(wb[q], 0x4140); a3 = u8x2_to_f16x2(wb[q], 0x4342);
                    } else {
                        a0 = wa[2 * q]; a2 = wa[2 * q + 1];
                        a1 = wb[2 * q]; a3 = wb[2 * q + 1];
                    }
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        if constexpr (W8) mma_f16(acc[rb][nt], a0, a1, a2, a3, xb[nt][2 * q], xb[nt][2 * q + 1]);
                        else mma_bf16(acc[rb][nt], a0, a1, a2, a3, xb[nt][2 * q], xb[nt][2 * q + 1]);
                    }
                }
            }
        }
    };

    // The weights do not depend on the kernel that precedes this one in the stream, the activations may: start the
    // weight stream (two stages into registers), let the next kernel in the stream begin its own, then wait for
    // the predecessor's results.
    issue(0, it_begin);
    issue(1, it_begin + 1);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int it = it_begin; it < it_end; it += 2) {
        const int it_in_chunk = (it - it_begin) % ITERS_PER_CHUNK;   // even: ITERS_PER_CHUNK is even
        if (it_in_chunk == 0) stage_x(it);
        multiply(0, it_in_chunk);
        issue(0, it + 2);
        if (it + 1 < it_end) multiply(1, it_in_chunk + 1);
        issue(1, it + 3);
    }

    if constexpr (W8) {
#pragma unroll
        for (int rb = 0; rb < 2; rb++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                acc[rb][nt][0] = scalbnf(acc[rb][nt][0], cur_e[nt][0]);
                acc[rb][nt][2] = scalbnf(acc[rb][nt][2], cur_e[nt][0]);
                acc[rb][nt][1] = scalbnf(acc[rb][nt][1], cur_e[nt][1]);
                acc[rb][nt][3] = scalbnf(acc[rb][nt][3], cur_e[nt][1]);
            }
    }
    // ---- partial tile -> shared memory: part[token][row] ----
    __syncthreads();
    float* part = (float*)smem;
#pragma unroll
    for (int rb = 0; rb < 2; rb++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const int row = warp * ROWS_PER_WARP + rb * 16 + g, tok = nt * 8 + 2 * t;
            part[tok * ROWS_PER_CTA + row] = acc[rb][nt][0];
            part[(tok + 1) * ROWS_PER_CTA + row] = acc[rb][nt][1];
            part[tok * ROWS_PER_CTA + row + 8] = acc[rb][nt][2];
            part[(tok + 1) * ROWS_PER_CTA + row + 8] = acc[rb][nt][3];
        }
    if (S > 1) cluster.sync(); else __syncthreads();

    // ---- reduce over splits in rank order, post-ops, store; the cluster's CTAs share the output elements ----
    const Epilogue& ep = p.ep;
    const bool silu = (ep.steps & B200FC_STEP_SILU_MUL) != 0;
    const int out_rows = silu ? ROWS_PER_CTA / 2 : ROWS_PER_CTA;
    const int total = out_rows * p.M;
    const int e_begin = (int)((long long)total * rank / S), e_end = (int)((long long)total * (rank + 1) / S);
    for (int e = e_begin + threadIdx.x; e < e_end; e += blockDim.x) {
        const int tok = e / out_rows, orow = e % out_rows;
        if (silu) {
            const int grow = 32 * (orow >> 4) + (orow & 15);
            float gsum = 0.0f, usum = 0.0f;
            for (int q = 0; q < S; q++) {
                const float* rp = S > 1 ? cluster.map_shared_rank(part, q) : part;
                gsum += rp[tok * ROWS_PER_CTA + grow];
                usum += rp[tok * ROWS_PER_CTA + grow + 16];
            }
            const int n_up = cta_row0 + grow + 16;
            if (n_up < p.n1) {
                const int nc = (cta_row0 >> 1) + orow;
                unsigned short* crow = (unsigned short*)((char*)ep.C + (long long)tok * ep.ldc);
                crow[nc] = f32_to_bf16_bits(silu_f(gsum) * usum);
            }
        } else {
            float sum = 0.0f;
            for (int q = 0; q < S; q++) {
                const float* rp = S > 1 ? cluster.map_shared_rank(part, q) : part;
                sum += rp[tok * ROWS_PER_CTA + orow];
            }
            const int n = cta_row0 + orow;
            if (n < p.n1) store_scalar(postop_scalar(sum, n, ep), tok, n, ep);
        }
    }
    if (S > 1) cluster.sync();  // nobody leaves while a peer may still read its partial tile
}

template <bool W8, int NT>
int launch_variant(const GemvParams& p, int row_ctas, cudaStream_t s) {
    constexpr int XROW = CHUNK_K * 2 + (W8 ? 16 : 64);
    constexpr int SMEM = 8 * NT * XROW + (W8 ? 8 * NT * (WARPS + 1) * 4 : 0);
    static_assert(SMEM >= ROWS_PER_CTA * 8 * NT * 4, "partial tile must fit the staging buffer");
    static std::atomic<unsigned long long> attr_devices{0};
    {
        const int arc = once_per_device(attr_devices, [] {
            B200FC_CUDA(cudaFuncSetAttribute(gemv_kernel<W8, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
            return (int)B200FC_OK;
        });
        if (arc) return arc;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(row_ctas, p.splits, 1);
    cfg.blockDim = dim3(WARPS * 32, 1, 1);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = p.splits;
    attr[0].val.clusterDim.z = 1;
    // programmatic dependent launch: this kernel may start while its predecessor in the stream drains; it reads
    // activations only after griddepcontrol.wait
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    B200FC_CUDA(cudaLaunchKernelEx(&cfg, gemv_kernel<W8, NT>, p));
    count_launch();
    return B200FC_OK;
}

}  // namespace

// B200FC_GEMV=regs selects the register-streaming kernel of this file, anything else the TMA-ring kernel (gemv_tma.cu)
static bool use_register_kernel() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("B200FC_GEMV");
        v = (e && e[0] == 'r') ? 1 : 0;
    }
    return v == 1;
}

int launch_gemv(const Weight& w, const void* A, int M, int K, int64_t lda, int n0, int n1, const Epilogue& ep,
                cudaStream_t s) {
    if (!use_register_kernel()) return launch_gemv_tma(w, A, M, K, lda, n0, n1, ep, s);
    if (M < 1 || M > 16) { set_error("gemv: M must be in [1, 16]"); return B200FC_ERR_INVALID; }
    if (w.dtype == B200FC_U8) { set_error("gemv: unsigned 8-bit weights are not supported with bf16 activations"); return B200FC_ERR_UNSUPPORTED; }
    if (n1 <= n0) return B200FC_OK;
    if ((ep.steps & B200FC_STEP_SILU_MUL) && (n0 % 32)) { set_error("gemv: SILU_MUL needs n0 %% 32 == 0"); return B200FC_ERR_INVALID; }
    GemvParams p;
    p.W = (const unsigned char*)w.data;
    p.ldw = w.ld_bytes();
    p.N_pad = w.N_pad;
    p.X = (const unsigned char*)A;
    p.ldx = lda;
    p.M = M; p.K = K;
    p.n_kb = (int)(w.ld_bytes() / KB_BYTES);
    p.n0 = n0; p.n1 = n1;
    p.ep = ep;
    const int row_ctas = (n1 - n0 + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
    const int iters_total = (p.n_kb + KB_PER_ITER - 1) / KB_PER_ITER;
    // split K over a cluster (at most 8 ways, the portable limit) while the whole grid still fits the GPU in one
    // wave (148 SMs x 4 resident CTAs) and every split keeps at least two pipeline stages of work
    int S = 1;
    while (S < 8 && row_ctas * S * 2 <= 148 * 4 && iters_total >= 4 * S) S *= 2;
    p.splits = S;
    const bool w8 = w.dtype == B200FC_S8;
    if (M <= 8) return w8 ? launch_variant<true, 1>(p, row_ctas, s) : launch_variant<false, 1>(p, row_ctas, s);
    return w8 ? launch_variant<true, 2>(p, row_ctas, s) : launch_variant<false, 2>(p, row_ctas, s);
}

}  // namespace b200fc
