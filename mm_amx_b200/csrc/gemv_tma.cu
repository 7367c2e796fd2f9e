// Decode-shaped fully-connected layer (M <= 16), weight stream fed by TMA into a shared-memory ring.
//
// Same contract and arithmetic as gemv.cu (the reference routines it replaces are listed there:
// amx_kernel::Matmul M <= 16 branches, include/kernels_amx.hpp:1216-1253 and 1381-1441,
// weight_compression/fc16m.cpp:451-502, fused-MLP decode tests/amx-mlp.cpp:648-737); what changes is how the bytes
// reach the multipliers.  Registers can hold only ~8 KB of weights in flight per warp, which leaves an SM short of
// the bytes in flight that 6.5 TB/s of HBM need.  Here one producer warp per CTA streams 16 KB stages (128 weight
// rows x 128 bytes of K, one 2-D TMA box with 128-byte swizzle) into a ring of 4-5 stages; with two CTAs per SM
// about 160 KB are in flight per SM and the stream never stops while the eight consumer warps stage activations,
// widen int8 weights or reduce.  Consumers copy their share of a stage (32 rows x 64 bytes of K: activation
// fragments are reused over two 16-row MMA blocks, which halves the shared-memory reads per weight) into registers
// (conflict-free through the swizzle), release the stage, and run the same mma.sync path as gemv.cu.
//   full[s]  : TMA complete_tx + one arrive.expect_tx by the producer        empty[s] : one arrive per consumer warp
// All mbarrier waits are bounded; on a time-out the CTA raises an abort flag, every role leaves its loop, the kernel
// stores an error code and still takes part in the cluster barriers.
#include <cooperative_groups.h>
#include <cuda.h>
#include <cuda_fp16.h>
#include "common.cuh"

namespace cg = cooperative_groups;

namespace b200fc {

namespace {

constexpr int CWARPS = 8;                       // consumer warps
constexpr int ROWS_PER_WARP = 32;               // a warp owns 32 rows x one 64-byte half of every stage
constexpr int ROWS_PER_CTA = (CWARPS / 2) * ROWS_PER_WARP;  // 128
constexpr int STAGE_K_BYTES = 128;              // bytes of K per row and stage (one swizzle atom)
constexpr int STAGE_BYTES = ROWS_PER_CTA * STAGE_K_BYTES;  // 16 KB
constexpr int CHUNK_K = 1024;                   // activation elements staged per chunk
constexpr int THREADS = (CWARPS + 1) * 32;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

struct Params {
    int n_stages_total;   // stages in a packed row (K_pad bytes / 128)
    const unsigned char* X;
    long long ldx;
    int M, K;
    int n0, n1;
    int splits;
    Epilogue ep;
    int* status;
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (globaltimer() - t0 > WAIT_LIMIT_NS) {
            *abort_flag = 1;
            return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, unsigned bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CWARPS * 32) : "memory"); }

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
// two offset-binary weights (bytes `sel` of w) -> f16x2 holding their values exactly (see gemv.cu)
__device__ __forceinline__ unsigned u8x2_to_f16x2(unsigned w, unsigned sel) {
    unsigned p = __byte_perm(w, 0x64646464u, sel);
    const __half2 off = __floats2half2_rn(1152.0f, 1152.0f);
    __half2 r = __hsub2(*(__half2*)&p, off);
    return *(unsigned*)&r;
}

template <bool W8, int NT> struct Layout {
    static constexpr int STAGES = NT == 1 ? 5 : 4;
    static constexpr int MP = 8 * NT;
    // bytes per staged activation row; the pad makes rows g and g + 1 fall into different bank halves for the
    // access pattern of each variant (see the fragment loads in the kernel)
    static constexpr int XROW = CHUNK_K * 2 + (W8 ? 64 : 16);
    static constexpr int RING = STAGES * STAGE_BYTES;
    static constexpr int X_OFF = RING;
    static constexpr int AUX_OFF = X_OFF + MP * XROW;          // smax [MP][CWARPS], sexp [MP]
    static constexpr int BAR_OFF = AUX_OFF + MP * (CWARPS + 1) * 4;
    static constexpr int SMEM = BAR_OFF + 2 * STAGES * 8 + 16 + 1024;  // + barriers, abort flag, alignment slack
};

template <bool W8, int NT>
__global__ void __launch_bounds__(THREADS, 2) gemv_tma_kernel(const __grid_constant__ CUtensorMap map_w, const Params p) {
    using L = Layout<W8, NT>;
    constexpr int MP = L::MP, XROW = L::XROW, STAGES = L::STAGES;
    constexpr int KE = W8 ? 128 : 64;                 // K elements per stage
    constexpr int STAGES_PER_CHUNK = CHUNK_K / KE;
    constexpr int MMA_PER_LOAD = W8 ? 4 : 2;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* xbuf = smem + L::X_OFF;
    unsigned* smax = (unsigned*)(smem + L::AUX_OFF);
    int* sexp = (int*)(smem + L::AUX_OFF + MP * CWARPS * 4);
    const unsigned bar_full = smem_u32(smem + L::BAR_OFF);
    const unsigned bar_empty = bar_full + STAGES * 8;
    volatile int* abort_flag = (volatile int*)(smem + L::BAR_OFF + 2 * STAGES * 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    cg::cluster_group cluster = cg::this_cluster();
    const int S = p.splits;
    const int rank = S > 1 ? (int)cluster.block_rank() : 0;
    const int it_begin = (int)((long long)p.n_stages_total * rank / S);
    const int it_end = (int)((long long)p.n_stages_total * (rank + 1) / S);
    const int cta_row0 = p.n0 + blockIdx.x * ROWS_PER_CTA;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; i++) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, CWARPS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // the next kernel in the stream may start its own weight stream now
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    constexpr int RB = ROWS_PER_WARP / 16;  // 16-row MMA blocks per warp
    float acc[RB][NT][4];
#pragma unroll
    for (int rb = 0; rb < RB; rb++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[rb][nt][i] = 0.0f;

    if (warp == CWARPS) {
        // ---------------- producer: weights never depend on the previous kernel, stream at once ----------------
        if (lane == 0) {
            int stage = 0;
            unsigned phase = 0;
            for (int it = it_begin; it < it_end; it++) {
                if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag)) break;
                mbar_expect_tx(bar_full + 8 * stage, STAGE_BYTES);
                tma_load_2d(smem_u32(smem + stage * STAGE_BYTES), &map_w, bar_full + 8 * stage, it * STAGE_K_BYTES, cta_row0);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else {
        // ---------------- consumers ----------------
        asm volatile("griddepcontrol.wait;" ::: "memory");  // activations may come from the previous kernel
        const int ctid = threadIdx.x;                        // 0 .. 127
        const bool x_vec = (((uintptr_t)p.X & 15) == 0) && ((p.ldx & 15) == 0);
        const int k_begin = it_begin * KE, k_end = it_end * KE;
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
        // Stages CHUNK_K activation elements of all MP rows: 128 sixteen-byte units per row, the 256 consumer
        // threads take two rows per pass.  All loads of a thread are issued before the first is converted / stored.
        constexpr int UNITS = CHUNK_K / 8;                    // 128
        constexpr int ROWS_PER_PASS = CWARPS * 32 / UNITS;    // 2
        constexpr int PASSES = MP / ROWS_PER_PASS;
        const int unit = ctid % UNITS, row0 = ctid / UNITS;
        // Compressed weights multiply fp16 x fp16, so every staged chunk is scaled per activation row by the power
        // of two that puts the row's largest magnitude (within the chunk) at 2^13 and converted to fp16: exact, since
        // fp16 keeps the 8-bit significand of bf16.  The accumulators carry the row's current scale (cur_e) and are
        // rescaled when a new chunk brings a different one; the scale is undone after the last stage.
        int cur_e[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) cur_e[nt][0] = cur_e[nt][1] = 0;
        auto stage_x = [&](int it) {
            const int k = it * KE + unit * 8;
            const bool need = k < k_end;
            consumer_sync();  // everyone is done with the previous chunk
            uint4 v[PASSES];
#pragma unroll
            for (int i = 0; i < PASSES; i++) v[i] = need ? load_x_unit(row0 + i * ROWS_PER_PASS, k) : make_uint4(0, 0, 0, 0);
            if constexpr (W8) {
#pragma unroll
                for (int i = 0; i < PASSES; i++) {
                    const unsigned w4[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
                    unsigned m = 0;
#pragma unroll
                    for (int q = 0; q < 4; q++) m = max(m, max(w4[q] & 0x7fffu, (w4[q] >> 16) & 0x7fffu));
                    m = __reduce_max_sync(0xffffffffu, m);
                    if (lane == 0) smax[(row0 + i * ROWS_PER_PASS) * CWARPS + warp] = m;   // 4 of the 8 slots per row
                }
                consumer_sync();
            }
#pragma unroll
            for (int i = 0; i < PASSES; i++) {
                const int row = row0 + i * ROWS_PER_PASS;
                uint4 o4 = v[i];
                if constexpr (W8) {
                    // the four warps that hold this row: warps 4 * row0 .. 4 * row0 + 3
                    unsigned m = 0;
#pragma unroll
                    for (int q = 0; q < 4; q++) m = max(m, smax[row * CWARPS + row0 * 4 + q]);
                    int field = (int)(m >> 7);          // biased exponent of the largest magnitude (bf16 layout)
                    field = field < 1 ? 1 : field;
                    int e = field - 127 - 13;
                    e = e < -126 ? -126 : e;
                    if (unit == 0) sexp[row] = e;
                    const float sc = __int_as_float((127 - e) << 23);  // 2^-e
                    const unsigned w4[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
                    unsigned o[4];
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        __half2 h = __floats2half2_rn(__uint_as_float(w4[q] << 16) * sc, __uint_as_float(w4[q] & 0xffff0000u) * sc);
                        o[q] = *(unsigned*)&h;
                    }
                    o4 = make_uint4(o[0], o[1], o[2], o[3]);
                }
                // compressed weights: the 16 units of a stage are stored transposed as a 4 x 4 grid, so that the
                // four lanes t of a fragment load (units 4t + i) touch four neighbouring 16-byte slots
                const int slot = W8 ? ((unit & ~15) | ((unit & 3) << 2) | ((unit >> 2) & 3)) : unit;
                if (need) *(uint4*)(xbuf + row * XROW + slot * 16) = o4;
            }
            consumer_sync();
            if constexpr (W8) {
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const int e0 = sexp[nt * 8 + 2 * t], e1 = sexp[nt * 8 + 2 * t + 1];
                    if (cur_e[nt][0] != e0 || cur_e[nt][1] != e1) {
#pragma unroll
                        for (int rb = 0; rb < RB; rb++) {
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

        int stage = 0;
        unsigned phase = 0;
        // byte offsets of this thread's 16-byte pieces inside a stage: rows (rb, h) -> warp*32 + rb*16 + h*8 + g,
        // logical chunk 2t + j, physical chunk = logical ^ (row & 7) = logical ^ g
        const int rg = warp >> 1, kh = warp & 1;       // row group (32 rows) and K half (64 bytes) of this warp
        const int row_base = rg * ROWS_PER_WARP + g;
        bool ok = true;
        for (int it = it_begin; it < it_end && ok; it++) {
            const int it_in_chunk = (it - it_begin) % STAGES_PER_CHUNK;
            if (it_in_chunk == 0) stage_x(it);
            if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) { ok = false; break; }
            uint4 w[RB][2];
            const unsigned char* sbase = smem + stage * STAGE_BYTES;
#pragma unroll
            for (int rb = 0; rb < RB; rb++)
#pragma unroll
                for (int h = 0; h < 2; h++)
                    w[rb][h] = *(const uint4*)(sbase + (row_base + rb * 16 + h * 8) * STAGE_K_BYTES + (((2 * t + kh) ^ g) << 4));
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * stage);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }

            {
                const int j = kh;
                // activations matching this thread's weight bytes: K elements [(2t + j) * (W8 ? 16 : 8), ...) of the stage
                const int xoff = W8 ? it_in_chunk * KE * 2 + (8 * j + t) * 16 : (it_in_chunk * KE + (2 * t + j) * 8) * 2;
                unsigned xb[NT][W8 ? 8 : 4];
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const unsigned char* xs = xbuf + (nt * 8 + g) * XROW + xoff;
                    uint4 a = *(const uint4*)xs;
                    xb[nt][0] = a.x; xb[nt][1] = a.y; xb[nt][2] = a.z; xb[nt][3] = a.w;
                    if constexpr (W8) {
                        uint4 b = *(const uint4*)(xs + 64);  // unit 4t + 2j + 1 sits four slots further
                        xb[nt][4] = b.x; xb[nt][5] = b.y; xb[nt][6] = b.z; xb[nt][7] = b.w;
                    }
                }
#pragma unroll
                for (int rb = 0; rb < RB; rb++) {
                    const unsigned wa[4] = {w[rb][0].x, w[rb][0].y, w[rb][0].z, w[rb][0].w};
                    const unsigned wb[4] = {w[rb][1].x, w[rb][1].y, w[rb][1].z, w[rb][1].w};
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
        }
        if constexpr (W8) {
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int rb = 0; rb < RB; rb++) {
                    acc[rb][nt][0] = scalbnf(acc[rb][nt][0], cur_e[nt][0]);
                    acc[rb][nt][2] = scalbnf(acc[rb][nt][2], cur_e[nt][0]);
                    acc[rb][nt][1] = scalbnf(acc[rb][nt][1], cur_e[nt][1]);
                    acc[rb][nt][3] = scalbnf(acc[rb][nt][3], cur_e[nt][1]);
                }
        }
    }

    // ---- partial tiles -> shared memory (over the activation buffer): part[K half][token][row] ----
    __syncthreads();
    float* part = (float*)xbuf;
    constexpr int PART_HALF = MP * ROWS_PER_CTA;  // floats per K half
    if (warp < CWARPS) {
        const int rg = warp >> 1, kh = warp & 1;
#pragma unroll
        for (int rb = 0; rb < RB; rb++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int row = rg * ROWS_PER_WARP + rb * 16 + g, tok = nt * 8 + 2 * t;
                float* pp = part + kh * PART_HALF;
                pp[tok * ROWS_PER_CTA + row] = acc[rb][nt][0];
                pp[(tok + 1) * ROWS_PER_CTA + row] = acc[rb][nt][1];
                pp[tok * ROWS_PER_CTA + row + 8] = acc[rb][nt][2];
                pp[(tok + 1) * ROWS_PER_CTA + row + 8] = acc[rb][nt][3];
            }
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, 3);
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
                gsum += rp[tok * ROWS_PER_CTA + grow] + rp[PART_HALF + tok * ROWS_PER_CTA + grow];
                usum += rp[tok * ROWS_PER_CTA + grow + 16] + rp[PART_HALF + tok * ROWS_PER_CTA + grow + 16];
            }
            if (cta_row0 + grow + 16 < p.n1) {
                unsigned short* crow = (unsigned short*)((char*)ep.C + (long long)tok * ep.ldc);
                crow[(cta_row0 >> 1) + orow] = f32_to_bf16_bits(silu_f(gsum) * usum);
            }
        } else {
            float sum = 0.0f;
            for (int q = 0; q < S; q++) {
                const float* rp = S > 1 ? cluster.map_shared_rank(part, q) : part;
                sum += rp[tok * ROWS_PER_CTA + orow] + rp[PART_HALF + tok * ROWS_PER_CTA + orow];
            }
            const int n = cta_row0 + orow;
            if (n < p.n1) store_scalar(postop_scalar(sum, n, ep), tok, n, ep);
        }
    }
    if (S > 1) cluster.sync();  // nobody leaves while a peer may still read its partial tile
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)sym;
    }
    return fn;
}

template <bool W8, int NT>
int launch_variant(const CUtensorMap& map, const Params& p, int row_ctas, cudaStream_t s) {
    using L = Layout<W8, NT>;
    static_assert(L::MP * L::XROW >= 2 * ROWS_PER_CTA * L::MP * 4, "partial tiles must fit the activation buffer");
    static std::atomic<unsigned long long> attr_devices{0};
    {
        const int arc = once_per_device(attr_devices, [] {
            B200FC_CUDA(cudaFuncSetAttribute(gemv_tma_kernel<W8, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM));
            return (int)B200FC_OK;
        });
        if (arc) return arc;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(row_ctas, p.splits, 1);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = L::SMEM;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = p.splits;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    B200FC_CUDA(cudaLaunchKernelEx(&cfg, gemv_tma_kernel<W8, NT>, map, p));
    count_launch();
    return B200FC_OK;
}

}  // namespace

int launch_gemv_tma(const Weight& w, const void* A, int M, int K, int64_t lda, int n0, int n1, const Epilogue& ep,
                    cudaStream_t s) {
    if (M < 1 || M > 16) { set_error("gemv: M must be in [1, 16]"); return B200FC_ERR_INVALID; }
    if (w.dtype == B200FC_U8) { set_error("gemv: unsigned 8-bit weights are not supported with bf16 activations"); return B200FC_ERR_UNSUPPORTED; }
    if (n1 <= n0) return B200FC_OK;
    if ((ep.steps & B200FC_STEP_SILU_MUL) && (n0 % 32)) { set_error("gemv: SILU_MUL needs n0 %% 32 == 0"); return B200FC_ERR_INVALID; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled entry point not available"); return B200FC_ERR_CUDA; }
    // the packed weights as a byte matrix [N_pad, K_pad bytes]; box = 128 bytes of K x 128 rows, 128-byte swizzle
    CUtensorMap map;
    cuuint64_t dims[2] = {(cuuint64_t)w.ld_bytes(), (cuuint64_t)w.N_pad};
    cuuint64_t strides[1] = {(cuuint64_t)w.ld_bytes()};
    cuuint32_t box[2] = {STAGE_K_BYTES, ROWS_PER_CTA};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w.data, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d)", (int)r); return B200FC_ERR_CUDA; }

    Params p;
    p.n_stages_total = (int)(w.ld_bytes() / STAGE_K_BYTES);
    p.X = (const unsigned char*)A;
    p.ldx = lda;
    p.M = M; p.K = K;
    p.n0 = n0; p.n1 = n1;
    p.ep = ep;
    p.status = kernel_status_word();
    const int row_ctas = (n1 - n0 + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
    // split K over a cluster (<= 8, the portable limit) while the grid still fits the GPU in one wave of two CTAs per
    // SM and every split keeps at least two stages
    int S = 1;
    while (S < 8 && row_ctas * S * 2 <= 148 * 2 && p.n_stages_total >= 4 * S) S *= 2;
    {
        static int forced = -1;  // B200FC_GEMV_SPLITS=1|2|4|8 (for experiments)
        if (forced < 0) {
            const char* e = getenv("B200FC_GEMV_SPLITS");
            forced = e ? atoi(e) : 0;
        }
        if ((forced == 1 || forced == 2 || forced == 4 || forced == 8) && p.n_stages_total >= 2 * forced) S = forced;
    }
    p.splits = S;
    const bool w8 = w.dtype == B200FC_S8;
    if (M <= 8) return w8 ? launch_variant<true, 1>(map, p, row_ctas, s) : launch_variant<false, 1>(map, p, row_ctas, s);
    return w8 ? launch_variant<true, 2>(map, p, row_ctas, s) : launch_variant<false, 2>(map, p, row_ctas, s);
}

}  // namespace b200fc
