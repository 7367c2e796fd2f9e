// Prefill-shaped fully-connected layer on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
// Replaces the M > 16 branches of amx_kernel::Matmul::operator() (kernel_2x2 over loop2D_opt_Mtail,
// include/kernels_amx.hpp:1255-1313) and the JIT 32x32 micro-kernel of the fused MLP (tests/amx-mlp.cpp:199-334),
// with PP::BiasGeluStore (kernels_amx.hpp:552-673) and the gate/up SiLU epilogue (tests/amx-mlp.cpp:716-734) fused
// behind the accumulator.
//
// Shape of the kernel
//   C tile 128 (M) x BN (N, 256 or 128); K advances in 128-byte slabs (64 bf16 / 128 int8).
//   A [M, K] (row-major, K contiguous) and the packed weights [N_pad, K_pad] (K contiguous) are both K-major, so a
//   2-D TMA box {128 bytes, rows} with 128-byte swizzle lands directly in the canonical tcgen05 operand layout.
//   One CTA per SM, persistent over tiles (m fastest, so CTAs running together share the same weight slab in L2).
//   Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer (one lane) and TMEM owner, warps 2-5 = epilogue.
//   The fp32 / int32 accumulator lives in TMEM, double buffered (2 x BN columns), so the epilogue of tile i
//   overlaps the main loop of tile i+1.
//   Tails: M and K tails come from TMA out-of-bounds zero fill, the N tail from zero rows of the packed weights;
//   stores are predicated.
// Every mbarrier wait is bounded: when one runs out, the CTA raises an abort flag, all roles fall through to the
// common exit (TMEM is freed there) and the kernel stores an error code for the host.
#include <cuda.h>
#include <cstdlib>
#include "common.cuh"

namespace b200fc {

namespace {

constexpr int BM = 128;
constexpr int SLAB_BYTES = 128;          // K extent of one pipeline stage, in bytes of operand elements
constexpr int MMA_K_BYTES = 32;          // K extent of one tcgen05.mma (16 bf16 / 32 int8)
constexpr int NUM_THREADS = 192;
constexpr int EPI_WARP0 = 2;
#ifndef B200FC_EPI_SLEEP_NS
#define B200FC_EPI_SLEEP_NS 256
#endif
constexpr int EPI_SLEEP_NS = B200FC_EPI_SLEEP_NS;

// staging tiles of the four epilogue warps: 32 rows x 32 four-byte columns each, rows padded to 33 words
constexpr int EPI_TILE_WORDS = 32 * 33;
constexpr int EPI_TILE_BYTES = 4 * EPI_TILE_WORDS * 4;

template <int BN> struct Cfg {
    static constexpr int STAGES = BN == 256 ? 4 : 6;
    static constexpr int A_BYTES = BM * SLAB_BYTES;
    static constexpr int B_BYTES = BN * SLAB_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TMEM_COLS = 2 * BN;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + EPI_TILE_BYTES;
};

struct GemmParams {
    int M, K, n0, n1;
    int tiles_m, tiles_n, k_slabs;
    unsigned idesc;
    int acc_is_int;
    int vec_ok;
    Epilogue ep;
    int* status;
    // split-K (2-CTA kernel): work item = (tile, split); with splits > 1 the epilogue stores raw accumulators into
    // slab `split` of a workspace ([splits][M][row pitch]) and a second kernel reduces and runs the post-ops
    int splits;
    long long split_stride;  // bytes between workspace slabs
    // 2-CTA kernel, splits == 1: > 0 = only the first item_limit tiles (in tile order) are computed by this launch; the
    // launcher hands the few tiles of a ragged last round to a second, K-split launch instead (launch_gemm_tc)
    int item_limit = 0;
    // 2-CTA kernel: > 0 = tiles are ordered in panels of this many row tiles (all column blocks of panel 0, then panel
    // 1, ...) and the activation loads carry an L2 evict-last hint, so that a panel of activations (panel_rows x 256 rows
    // x K) stays in L2 while the weights stream past it; 0 = one panel (row tile fastest over the whole M)
    int panel_rows = 0;
    // Fused tensor-parallel all-reduce (2-CTA kernel, ar_world > 0).  The epilogue stores this rank's bf16 tile into
    // its replica of a symmetric "partial" buffer (ep.C) and bumps the tile's arrival counter on the tile's owner
    // rank; the last CTA pairs of the grid do not multiply but reduce the tiles this rank owns.
    int ar_world, ar_rank;
    int ar_phases;              // bit 0: multiply, bit 1: reduce (both set in normal use; single bits for measurements)
    int ar_gemm_pairs;          // pairs that multiply; pairs beyond reduce from the start
    int ar_work_counter;        // index, in this rank's counter array, of the counter that hands out reduction units
    unsigned ar_target;         // arrivals that mean "every rank has stored these 128 rows of the tile" (world x 4 epilogue warps)
    unsigned* ar_flags[8];      // ar_flags[r]: arrival counters of rank r (peer-mapped), two per tile (one per CTA of the pair)
    const char* ar_partial_mc;  // multicast address of all replicas of the partial buffer
    char* ar_out_mc;            // multicast address of all replicas of the output buffer
    unsigned long long wait_limit_ns;  // every bounded wait gives up after this long
};

// ---- PTX wrappers ------------------------------------------------------------------------------------------------
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
// Bounded wait.  Returns false when the CTA is aborting (this wait or another role's ran out of time).
// SLEEP_NS > 0: back off between polls (for waits that are long and not latency critical: the epilogue warps wait most
// of a tile's main loop, and five spinning warps cost issue slots and power that the tensor pipe could use).
template <int SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag, unsigned long long limit) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer();
    while (true) {
        if (SLEEP_NS > 0) __nanosleep(SLEEP_NS);
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (globaltimer() - t0 > limit) {
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
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
template <bool I8>
__device__ __forceinline__ void tc_mma(unsigned d_tmem, unsigned long long adesc, unsigned long long bdesc,
                                       unsigned idesc, unsigned accumulate) {
    if constexpr (I8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
__device__ __forceinline__ void tc_ld32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory operand descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes
// apart (stride-dimension byte offset); descriptor version 1 (Blackwell).
__device__ __forceinline__ unsigned long long make_smem_desc(unsigned smem_addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)1 << 16;            // leading-dimension byte offset (unused for swizzled K-major)
    d |= (unsigned long long)(1024 >> 4) << 32;  // stride-dimension byte offset
    d |= (unsigned long long)1 << 46;            // descriptor version
    d |= (unsigned long long)2 << 61;            // SWIZZLE_128B
    return d;
}

// ---- epilogue on 32 consecutive columns of one output row ------------------------------------------------------------
struct EpiArgs {       // what the epilogue of one 32-column chunk needs to know
    const Epilogue* ep;
    int vec_ok, acc_is_int, n1;
    int M;             // rows of the output
    unsigned* tile;    // this warp's staging tile in shared memory (EPI_TILE_WORDS words)
    // the chunk's 32 per-column values, staged in shared memory ahead of the tile (16-byte aligned), or null: read
    // them from global memory
    const float* cv_deq = nullptr;
    const float* cv_bias = nullptr;
    const float* cv_q = nullptr;
};
// 32 rows x 32 four-byte values, one row per lane in registers -> global memory with full-line stores: the tile goes
// through shared memory and comes back with eight lanes per row (16 bytes each), so that one store instruction writes
// four whole 128-byte row segments instead of 32 scattered 16-byte pieces.  Both passes use 16-byte accesses: row r
// keeps its 16-byte piece j at position j ^ (r & 7), which makes the eight lanes of every shared-memory wavefront hit
// eight different bank groups on the way in (lanes = rows) and on the way out (lanes = pieces of one row).
// Called by all lanes of the warp; `tile` is 16-byte aligned.
__device__ __forceinline__ void store_tile_4b(const unsigned (&val)[32], unsigned* tile, char* C, long long ldc, int m, int n,
                                              int M) {
    const int lane = threadIdx.x & 31, m0 = m - lane;
    uint4* t4 = (uint4*)tile;
#pragma unroll
    for (int j = 0; j < 8; j++)
        t4[lane * 8 + (j ^ (lane & 7))] = make_uint4(val[4 * j], val[4 * j + 1], val[4 * j + 2], val[4 * j + 3]);
    __syncwarp();
    const int piece = lane & 7;
#pragma unroll
    for (int it = 0; it < 8; it++) {
        const int rr = it * 4 + (lane >> 3);
        const uint4 q = t4[rr * 8 + (piece ^ (rr & 7))];
        if (m0 + rr < M) *(uint4*)(C + (long long)(m0 + rr) * ldc + (long long)(n + piece * 4) * 4) = q;
    }
    __syncwarp();
}
// the 32 per-column values vec[n .. n + 32) of a chunk (every lane needs all of them): eight 16-byte loads when the
// chunk is whole and the vector 16-byte aligned, else 32 scalar loads clamped to the last valid column
__device__ __forceinline__ void load_col_vec(const float* __restrict__ vec, int n, int n1, float (&out)[32]) {
    if (n + 32 <= n1 && (((uintptr_t)(vec + n)) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float4 t = __ldg((const float4*)(vec + n) + j);
            out[4 * j] = t.x; out[4 * j + 1] = t.y; out[4 * j + 2] = t.z; out[4 * j + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; j++) out[j] = __ldg(vec + min(n + j, n1 - 1));
    }
}
// the same 32 values from the warp's staged copy (every lane reads the same addresses: broadcasts)
__device__ __forceinline__ void load_col_vec(const float* staged, const float* __restrict__ vec, int n, int n1, float (&out)[32]) {
    if (staged) {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float4 t = ((const float4*)staged)[j];
            out[4 * j] = t.x; out[4 * j + 1] = t.y; out[4 * j + 2] = t.z; out[4 * j + 3] = t.w;
        }
    } else {
        load_col_vec(vec, n, n1, out);
    }
}
__device__ __forceinline__ void epilogue_chunk(const unsigned (&r)[32], int m, int n, const EpiArgs p, bool row_ok,
                                               long long c_offset = 0) {
    const Epilogue& ep = *p.ep;
    const bool staged = p.vec_ok && n + 32 <= p.n1 && !ep.mc_reduce;   // warp-uniform
    if (ep.out_dtype == B200FC_S32 && staged) {
        store_tile_4b(r, p.tile, (char*)ep.C + c_offset, ep.ldc, m, n, p.M);
        return;
    }
    const bool staged_f32 = ep.out_dtype == B200FC_F32 && staged && !(ep.steps & B200FC_STEP_SILU_MUL);   // warp-uniform
    if (!row_ok && !staged_f32) return;   // (rows beyond M take part in the staged store's shuffle through shared memory)
    char* crow = (char*)ep.C + c_offset + (long long)m * ep.ldc;
    if (ep.out_dtype == B200FC_S32) {  // raw accumulators
        if (p.vec_ok && n + 32 <= p.n1) {
            int4* dst = (int4*)(crow + (long long)n * 4);
#pragma unroll
            for (int j = 0; j < 8; j++) dst[j] = make_int4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        } else {
            for (int j = 0; j < 32; j++)
                if (n + j < p.n1) ((int*)crow)[n + j] = (int)r[j];
        }
        return;
    }
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; j++) v[j] = p.acc_is_int ? (float)(int)r[j] : __uint_as_float(r[j]);

    if (ep.mc_reduce) {
        // Fused all-reduce: C is a multicast mapping of the output on every GPU of the tensor-parallel group; the
        // NVSwitch adds this rank's contribution into all replicas (multimem.red), so no separate collective runs.
        const bool full = p.vec_ok && n + 32 <= p.n1;
        if (ep.out_dtype == B200FC_F32) {
            float* dst = (float*)(crow + (long long)n * 4);
            if (full) {
#pragma unroll
                for (int j = 0; j < 8; j++)
                    asm volatile("multimem.red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4 * j),
                                 "f"(v[4 * j]), "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                                 : "memory");
            } else {
                for (int j = 0; j < 32; j++)
                    if (n + j < p.n1) asm volatile("multimem.red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(dst + j), "f"(v[j]) : "memory");
            }
        } else {
            unsigned short* dst = (unsigned short*)(crow + (long long)n * 2);
            if (full) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    unsigned o[4];
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * j + 2 * q], v[8 * j + 2 * q + 1]);
                        o[q] = *(unsigned*)&h;
                    }
                    asm volatile("multimem.red.relaxed.sys.global.add.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst + 8 * j),
                                 "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                                 : "memory");
                }
            } else {
                for (int j = 0; j < 32; j += 2)   // the launcher guarantees an even column range for this mode
                    if (n + j + 1 < p.n1) {
                        __nv_bfloat162 h = __floats2bfloat162_rn(v[j], v[j + 1]);
                        asm volatile("multimem.red.relaxed.sys.global.add.bf16x2 [%0], %1;" ::"l"(dst + j), "r"(*(unsigned*)&h) : "memory");
                    }
            }
        }
        return;
    }

    if (ep.steps & B200FC_STEP_SILU_MUL) {
        // columns [0,16) gate, [16,32) up of the same 16 channels -> 16 bf16 outputs at column n/2
        __align__(16) unsigned short o[16];
#pragma unroll
        for (int j = 0; j < 16; j++) o[j] = f32_to_bf16_bits(silu_f(v[j]) * v[16 + j]);
        int nc = n >> 1;
        unsigned short* dst = (unsigned short*)crow + nc;
        if (p.vec_ok && n + 32 <= p.n1) {
            ((int4*)dst)[0] = *(int4*)&o[0];
            ((int4*)dst)[1] = *(int4*)&o[8];
        } else {
            for (int j = 0; j < 16; j++)
                if (n + 16 + j < p.n1) dst[j] = o[j];
        }
        return;
    }

    if (ep.steps & B200FC_STEP_DEQUANT) {
        if (ep.deq_per_oc) {
            float sc[32];
            load_col_vec(p.cv_deq, ep.deq_per_oc, n, p.n1, sc);
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] *= ep.deq_scale * sc[j];
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] *= ep.deq_scale;
        }
    }
    if (ep.steps & B200FC_STEP_BIAS) {
        float bs[32];
        load_col_vec(p.cv_bias, ep.bias, n, p.n1, bs);
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] += bs[j];
    }
    if (ep.steps & B200FC_STEP_GELU) {
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] = gelu_erf_poly(v[j]);
    }
    if (ep.steps & B200FC_STEP_QUANT) {
        if (ep.q_per_oc) {
            float qs[32];
            load_col_vec(p.cv_q, ep.q_per_oc, n, p.n1, qs);
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] *= qs[j];
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] *= ep.q_scale;
        }
    }
    const bool full = p.vec_ok && n + 32 <= p.n1;
    if (ep.residual && row_ok) {
        // residual added in fp32, before the one rounding of the output
        const char* rrow = (const char*)ep.residual + (long long)m * ep.ld_res;
        if (full && (((uintptr_t)rrow + (size_t)n * 2) & 15) == 0) {
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int4 t = __ldg((const int4*)(rrow + (long long)n * 2) + q);
                const unsigned w4[4] = {(unsigned)t.x, (unsigned)t.y, (unsigned)t.z, (unsigned)t.w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    v[8 * q + 2 * e] += __uint_as_float(w4[e] << 16);
                    v[8 * q + 2 * e + 1] += __uint_as_float(w4[e] & 0xffff0000u);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++)
                v[j] += __uint_as_float((unsigned)((const unsigned short*)rrow)[min(n + j, p.n1 - 1)] << 16);
        }
    }
    if (staged_f32) {
        unsigned u[32];
#pragma unroll
        for (int j = 0; j < 32; j++) u[j] = __float_as_uint(v[j]);
        store_tile_4b(u, p.tile, (char*)ep.C + c_offset, ep.ldc, m, n, p.M);
    } else if (ep.out_dtype == B200FC_F32) {
        if (full) {
            float4* dst = (float4*)(crow + (long long)n * 4);
#pragma unroll
            for (int j = 0; j < 8; j++) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
            for (int j = 0; j < 32; j++)
                if (n + j < p.n1) ((float*)crow)[n + j] = v[j];
        }
    } else if (ep.out_dtype == B200FC_BF16) {
        if (full) {
            __align__(16) unsigned o[16];
#pragma unroll
            for (int j = 0; j < 16; j++) {
                __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                o[j] = *(unsigned*)&h;
            }
            int4* dst = (int4*)(crow + (long long)n * 2);
#pragma unroll
            for (int j = 0; j < 4; j++) dst[j] = *(int4*)&o[4 * j];
        } else {
            for (int j = 0; j < 32; j++)
                if (n + j < p.n1) ((unsigned short*)crow)[n + j] = f32_to_bf16_bits(v[j]);
        }
    } else {  // int8
        if (full) {
            __align__(16) unsigned o[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                unsigned b0 = f32_to_s8(v[4 * j]) & 0xff, b1 = f32_to_s8(v[4 * j + 1]) & 0xff;
                unsigned b2 = f32_to_s8(v[4 * j + 2]) & 0xff, b3 = f32_to_s8(v[4 * j + 3]) & 0xff;
                o[j] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
            }
            int4* dst = (int4*)(crow + n);
            dst[0] = *(int4*)&o[0];
            dst[1] = *(int4*)&o[4];
        } else {
            for (int j = 0; j < 32; j++)
                if (n + j < p.n1) ((signed char*)crow)[n + j] = (signed char)f32_to_s8(v[j]);
        }
    }
}

// ---- the kernel --------------------------------------------------------------------------------------------------------
template <int BN, bool I8>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const GemmParams p) {
    using C = Cfg<BN>;
    extern __shared__ unsigned char smem_raw[];
    // operand stages need 1024-byte alignment (128-byte swizzle atom = 8 rows x 128 bytes)
    // (pointer arithmetic on the __shared__ array, not an integer round trip: the accesses stay shared-space loads / stores)
    unsigned char* smem = smem_raw + (((smem_u32(smem_raw) + 1023u) & ~1023u) - smem_u32(smem_raw));
    unsigned long long* bars = (unsigned long long*)(smem + C::STAGES * C::STAGE_BYTES);
    // barrier slots: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    const unsigned bar_full = smem_u32(bars);
    const unsigned bar_empty = smem_u32(bars + C::STAGES);
    const unsigned bar_acc_full = smem_u32(bars + 2 * C::STAGES);
    const unsigned bar_acc_empty = smem_u32(bars + 2 * C::STAGES + 2);
    unsigned* tmem_holder = (unsigned*)(bars + 2 * C::STAGES + 4);
    volatile int* abort_flag = (volatile int*)(tmem_holder + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int i = 0; i < C::STAGES; i++) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(bar_acc_full + 8 * i, 1);
            mbar_init(bar_acc_empty + 8 * i, 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                     "r"((unsigned)C::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_holder;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            unsigned phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
                const int row_a = tm * BM, row_w = p.n0 + tn * BN;
                for (int ks = 0; ks < p.k_slabs; ks++) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.wait_limit_ns)) { ok = false; break; }
                    const unsigned full = bar_full + 8 * stage;
                    mbar_expect_tx(full, C::STAGE_BYTES);
                    const unsigned sa = smem_u32(smem + stage * C::STAGE_BYTES);
                    const int kx = ks * (I8 ? SLAB_BYTES : SLAB_BYTES / 2);  // element coordinate along K
                    tma_load_2d(sa, &map_a, full, kx, row_a);
                    tma_load_2d(sa + C::A_BYTES, &map_w, full, kx, row_w);
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        int stage = 0;
        unsigned phase = 0;
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, it++) {
            const int ab = it & 1;
            const unsigned acc_phase = (unsigned)(it >> 1) & 1;
            if (!mbar_wait(bar_acc_empty + 8 * ab, acc_phase ^ 1, abort_flag, p.wait_limit_ns)) { ok = false; break; }
            tc_fence_after();
            const unsigned d_tmem = tmem_base + (unsigned)(ab * BN);
            for (int ks = 0; ks < p.k_slabs; ks++) {
                if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.wait_limit_ns)) { ok = false; break; }
                tc_fence_after();
                if (lane == 0) {
                    const unsigned sa = smem_u32(smem + stage * C::STAGE_BYTES);
                    const unsigned long long adesc = make_smem_desc(sa);
                    const unsigned long long bdesc = make_smem_desc(sa + C::A_BYTES);
#pragma unroll
                    for (int k = 0; k < SLAB_BYTES / MMA_K_BYTES; k++) {
                        // advancing K inside the swizzle atom = advancing the start address (units of 16 bytes)
                        tc_mma<I8>(d_tmem, adesc + (unsigned long long)(k * (MMA_K_BYTES >> 4)),
                                   bdesc + (unsigned long long)(k * (MMA_K_BYTES >> 4)), p.idesc,
                                   (unsigned)((ks | k) != 0));
                    }
                    tc_commit(bar_empty + 8 * stage);  // frees the stage once these MMAs have read it
                    if (ks == p.k_slabs - 1) tc_commit(bar_acc_full + 8 * ab);
                }
                __syncwarp();
                if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else {
        // ---------------- epilogue warps ----------------
        const int quarter = warp & 3;  // TMEM lanes this warp may read: [32*quarter, 32*quarter + 32)
        unsigned* epi_tile = (unsigned*)(smem + C::STAGES * C::STAGE_BYTES + 256) + quarter * EPI_TILE_WORDS;
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, it++) {
            const int ab = it & 1;
            const unsigned acc_phase = (unsigned)(it >> 1) & 1;
            const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
            if (!mbar_wait<EPI_SLEEP_NS>(bar_acc_full + 8 * ab, acc_phase, abort_flag, p.wait_limit_ns)) { ok = false; break; }
            tc_fence_after();
            const int m = tm * BM + quarter * 32 + lane;
            const bool row_ok = m < p.M;
            const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(ab * BN);
#pragma unroll 1
            for (int c = 0; c < BN / 32; c++) {
                const int n = p.n0 + tn * BN + c * 32;
                if (n >= p.n1) break;  // warp-uniform
                unsigned r[32];
                tc_ld32(taddr + (unsigned)(c * 32), r);
                tc_wait_ld();
                epilogue_chunk(r, m, n, EpiArgs{&p.ep, p.vec_ok, p.acc_is_int, p.n1, p.M, epi_tile}, row_ok);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + 8 * ab);
        }
    }

    // ---------------- common exit ----------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // give copies that may still be in flight time to land before shared memory is released
        if (threadIdx.x == 0) {
            atomicExch(p.status, 1);
            const unsigned long long t0 = globaltimer();
            while (globaltimer() - t0 < 200000ull) { }
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)C::TMEM_COLS)
                     : "memory");
    }
}

// ---- the 2-CTA kernel ---------------------------------------------------------------------------------------------
// A pair of CTAs (a cluster of two, on neighbouring SMs) computes one 256 (M) x BN tile with cta_group::2 MMAs.
// Each CTA stages its own 128 rows of A and only HALF of the weight rows of the tile (BN / 2), so a stage is
// 16 KB + BN/2 * 128 B instead of 16 KB + BN * 128 B: a third fewer operand bytes cross L2 -> shared memory per flop,
// which is what bounds the 1-CTA kernel.  The leader CTA (cluster rank 0) issues the MMAs for both; its TMEM and
// the peer's each hold the 128 x BN accumulator rows of their own half of M.
//   full[s]       lives in the leader: one arrive.expect_tx by the leader's producer for the bytes of BOTH CTAs;
//                 the peer's TMA loads complete_tx on the leader's barrier (cta_group::2 loads, no multicast).
//   empty[s]      one per CTA, released by the leader's tcgen05.commit multicast to both CTAs.
//   acc_full[b]   one per CTA, same multicast commit after the last K slab.
//   acc_empty[b]  lives in the leader, 8 arrivals: the four epilogue warps of each CTA (the peer's arrive remotely).
// Cluster barriers bracket the kernel so that neither CTA touches the other's barriers before they exist or
// after it has exited.  All mbarrier waits are bounded as in the 1-CTA kernel.
template <int BN> struct Cfg2 {
    static constexpr int STAGES = BN == 256 ? 6 : 8;
    static constexpr int A_BYTES = BM * SLAB_BYTES;
    static constexpr int B_BYTES = (BN / 2) * SLAB_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TMEM_COLS = 2 * BN;
    // per epilogue warp: the tile's per-column vectors (dequantisation scales, bias, quantisation scales)
    static constexpr int COLVEC_BYTES = 4 * 3 * BN * 4;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + EPI_TILE_BYTES + COLVEC_BYTES;
};

__device__ __forceinline__ unsigned cluster_ctarank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ unsigned mapa_rank(unsigned addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_remote(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(unsigned dst, const CUtensorMap* map, unsigned leader_bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(leader_bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair_keep(unsigned dst, const CUtensorMap* map, unsigned leader_bar, int x, int y,
                                                      unsigned long long policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"(map), "r"(leader_bar), "r"(x), "r"(y), "l"(policy)
        : "memory");
}
// tile index (the order in which the CTA pairs take tiles) -> row tile tm and column tile tn
__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& tm, int& tn) {
    if (p.panel_rows <= 0 || p.panel_rows >= p.tiles_m) {
        tm = tile % p.tiles_m; tn = tile / p.tiles_m;
    } else {
        const int per_panel = p.panel_rows * p.tiles_n;
        const int pi = tile / per_panel, r = tile - pi * per_panel;
        const int ph = min(p.panel_rows, p.tiles_m - pi * p.panel_rows);   // the last panel may be shorter
        tm = pi * p.panel_rows + r % ph; tn = r / ph;
    }
}
__device__ __forceinline__ void tc_commit_pair(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((unsigned short)3)
                 : "memory");
}
template <bool I8>
__device__ __forceinline__ void tc_mma_pair(unsigned d_tmem, unsigned long long adesc, unsigned long long bdesc,
                                            unsigned idesc, unsigned accumulate) {
    if constexpr (I8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

constexpr int AR_UNROLL = 22;  // 192 threads x 22 pieces cover the 4096 pieces of a 128 x 256 bf16 unit

// All-reduce work of the fused tensor-parallel down projection, run by whole CTAs: the pairs reserved for it from the
// start of the kernel and every multiplying CTA once its own tiles are done.
// Tile t belongs to rank t % world.  Unit of work: the 128 rows of an owned tile that one CTA of a multiplying pair
// produced (own arrival counter); units are claimed in tile order from a counter in this rank's memory.  Once every
// rank has stored its bf16 contribution (arrival counter reached), the unit is pulled from all replicas with
// multimem.ld_reduce — the NVSwitch adds them, accumulating in fp32 — and the sum is written to every rank's output
// with multimem.st.  So each contribution crosses NVLink once, while the multiplying pairs are busy with later
// tiles.  A whole unit (<= 4096 16-byte pieces) is in flight at once, AR_UNROLL reductions per thread, because a trip
// through the switch takes microseconds.
template <int BN>
__device__ void allreduce_units(const GemmParams& p, int num_tiles, volatile int* unit_slot, volatile int* abort_flag) {
    unsigned* my_flags = p.ar_flags[p.ar_rank];
    const int owned = (num_tiles - p.ar_rank + p.ar_world - 1) / p.ar_world;
    const int n_units = 2 * owned;
    while (true) {
        if (threadIdx.x == 0) *unit_slot = (int)atomicAdd(my_flags + p.ar_work_counter, 1u);
        __syncthreads();
        const int u = *unit_slot;
        if (u >= n_units) break;
        const int tile = p.ar_rank + (u >> 1) * p.ar_world, half = u & 1;
        int tm, tn;
        tile_coords(p, tile, tm, tn);
        const int r0 = tm * (2 * BM) + half * BM, c0 = p.n0 + tn * BN;
        const int rows = min(BM, p.M - r0), cols = min(BN, p.n1 - c0);
        if (threadIdx.x == 0 && rows > 0) {
            const unsigned long long t0 = globaltimer();
            while (true) {
                unsigned v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(my_flags + 2 * tile + half) : "memory");
                if (v >= p.ar_target) break;
                if (globaltimer() - t0 > p.wait_limit_ns) { *abort_flag = 1; break; }
            }
        }
        // Thread 0's acquire load and the CTA barrier order every thread's loads below after the arrivals; a
        // system-scope fence here would also wait for this thread's multicast stores of the previous unit to reach
        // every GPU (measured: 8 us per unit).  The barrier also keeps unit_slot from being rewritten too early.
        __syncthreads();
        if (*abort_flag) break;
        if (rows <= 0) continue;
        const int ppr = cols >> 3;  // 16-byte pieces (8 bf16) per row
        const int total = rows * ppr;
        const long long base_off = (long long)r0 * p.ep.ldc + (long long)c0 * 2;
        for (int base = threadIdx.x; base < total; base += NUM_THREADS * AR_UNROLL) {
            unsigned v[AR_UNROLL][4];
#pragma unroll
            for (int k = 0; k < AR_UNROLL; k++) {
                const int i = base + k * NUM_THREADS;
                const int row = i / ppr, pc = i - row * ppr;
                const long long off = base_off + (long long)row * p.ep.ldc + pc * 16;
                if (i < total)
                    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(v[k][0]), "=r"(v[k][1]), "=r"(v[k][2]), "=r"(v[k][3])
                                 : "l"(p.ar_partial_mc + off)
                                 : "memory");
            }
#pragma unroll
            for (int k = 0; k < AR_UNROLL; k++) {
                const int i = base + k * NUM_THREADS;
                const int row = i / ppr, pc = i - row * ppr;
                const long long off = base_off + (long long)row * p.ep.ldc + pc * 16;
                if (i < total)
                    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(p.ar_out_mc + off),
                                 "r"(v[k][0]), "r"(v[k][1]), "r"(v[k][2]), "r"(v[k][3])
                                 : "memory");
            }
        }
    }
}

template <int BN, bool I8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                const GemmParams p) {
    using C = Cfg2<BN>;
    extern __shared__ unsigned char smem_raw[];
    // (pointer arithmetic on the __shared__ array, not an integer round trip: the accesses stay shared-space loads / stores)
    unsigned char* smem = smem_raw + (((smem_u32(smem_raw) + 1023u) & ~1023u) - smem_u32(smem_raw));
    unsigned long long* bars = (unsigned long long*)(smem + C::STAGES * C::STAGE_BYTES);
    const unsigned bar_full = smem_u32(bars);
    const unsigned bar_empty = smem_u32(bars + C::STAGES);
    const unsigned bar_acc_full = smem_u32(bars + 2 * C::STAGES);
    const unsigned bar_acc_empty = smem_u32(bars + 2 * C::STAGES + 2);
    unsigned* tmem_holder = (unsigned*)(bars + 2 * C::STAGES + 4);
    volatile int* abort_flag = (volatile int*)(tmem_holder + 1);
    volatile int* unit_slot = (volatile int*)(tmem_holder + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, grid_pairs = gridDim.x >> 1;
    const int num_pairs = p.ar_world ? p.ar_gemm_pairs : grid_pairs;  // pairs that take part in the multiplication
    const bool comm_role = p.ar_world && pair >= num_pairs;
    const int num_tiles = p.tiles_m * p.tiles_n;  // tiles of 256 x BN
    const int num_items = p.item_limit > 0 ? p.item_limit : num_tiles * p.splits;   // (tile, K split) work items

    if (threadIdx.x == 0) {
        for (int i = 0; i < C::STAGES; i++) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(bar_acc_full + 8 * i, 1);
            mbar_init(bar_acc_empty + 8 * i, 8);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                     "r"((unsigned)C::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before anyone signals them
    tc_fence_after();
    // a kernel launched as a programmatic dependent (the split-K reduction) may become resident from here on
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const unsigned tmem_base = *tmem_holder;

    if (comm_role) {
        // ---------------- all-reduce role (whole CTA) ----------------
        if (p.ar_phases & 2) allreduce_units<BN>(p, num_tiles, unit_slot, abort_flag);
    } else if (p.ar_world && !(p.ar_phases & 1)) {
    } else if (warp == 0) {
        // ---------------- TMA producer (one per CTA) ----------------
        if (lane == 0) {
            int stage = 0;
            unsigned phase = 0;
            bool ok = true;
            const unsigned leader_full = mapa_rank(bar_full, 0);
            unsigned long long keep_policy = 0;
            if (p.panel_rows > 0) asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(keep_policy));
            for (int item = pair; item < num_items && ok; item += num_pairs) {
                const int tile = item % num_tiles, split = item / num_tiles;
                const int ks0 = p.k_slabs * split / p.splits, ks1 = p.k_slabs * (split + 1) / p.splits;
                int tm, tn;
                tile_coords(p, tile, tm, tn);
                const int row_a = tm * (2 * BM) + (int)rank * BM;
                const int row_w = p.n0 + tn * BN + (int)rank * (BN / 2);
                for (int ks = ks0; ks < ks1; ks++) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.wait_limit_ns)) { ok = false; break; }
                    if (leader) mbar_expect_tx(bar_full + 8 * stage, 2 * C::STAGE_BYTES);
                    const unsigned sa = smem_u32(smem + stage * C::STAGE_BYTES);
                    const int kx = ks * (I8 ? SLAB_BYTES : SLAB_BYTES / 2);
                    if (p.panel_rows > 0) tma_load_2d_pair_keep(sa, &map_a, leader_full + 8 * stage, kx, row_a, keep_policy);
                    else tma_load_2d_pair(sa, &map_a, leader_full + 8 * stage, kx, row_a);
                    tma_load_2d_pair(sa + C::A_BYTES, &map_w, leader_full + 8 * stage, kx, row_w);
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only; one thread waits and issues, its warp mates park) ----------------
        if (leader && lane == 0) {
            int stage = 0;
            unsigned phase = 0;
            int it = 0;
            bool ok = true;
            for (int item = pair; item < num_items && ok; item += num_pairs, it++) {
                const int split = item / num_tiles;
                const int ks0 = p.k_slabs * split / p.splits, ks1 = p.k_slabs * (split + 1) / p.splits;
                const int ab = it & 1;
                const unsigned acc_phase = (unsigned)(it >> 1) & 1;
                if (!mbar_wait(bar_acc_empty + 8 * ab, acc_phase ^ 1, abort_flag, p.wait_limit_ns)) { ok = false; break; }
                tc_fence_after();
                const unsigned d_tmem = tmem_base + (unsigned)(ab * BN);
                for (int ks = ks0; ks < ks1; ks++) {
                    if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.wait_limit_ns)) { ok = false; break; }
                    tc_fence_after();
                    const unsigned sa = smem_u32(smem + stage * C::STAGE_BYTES);
                    const unsigned long long adesc = make_smem_desc(sa);
                    const unsigned long long bdesc = make_smem_desc(sa + C::A_BYTES);
#pragma unroll
                    for (int k = 0; k < SLAB_BYTES / MMA_K_BYTES; k++)
                        tc_mma_pair<I8>(d_tmem, adesc + (unsigned long long)(k * (MMA_K_BYTES >> 4)),
                                        bdesc + (unsigned long long)(k * (MMA_K_BYTES >> 4)), p.idesc,
                                        (unsigned)(((ks - ks0) | k) != 0));
                    tc_commit_pair(bar_empty + 8 * stage);
                    if (ks == ks1 - 1) tc_commit_pair(bar_acc_full + 8 * ab);
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue warps (both CTAs, own 128 rows) ----------------
        const int quarter = warp & 3;
        unsigned* epi_tile = (unsigned*)(smem + C::STAGES * C::STAGE_BYTES + 256) + quarter * EPI_TILE_WORDS;
        float* colvec = (float*)(smem + C::STAGES * C::STAGE_BYTES + 256 + EPI_TILE_BYTES) + quarter * 3 * BN;
        const bool plain_ep = !(p.ep.steps & B200FC_STEP_SILU_MUL) && !p.ep.mc_reduce && p.ep.out_dtype != B200FC_S32;
        const bool use_deq = plain_ep && (p.ep.steps & B200FC_STEP_DEQUANT) && p.ep.deq_per_oc;
        const bool use_bias = plain_ep && (p.ep.steps & B200FC_STEP_BIAS) && p.ep.bias;
        const bool use_q = plain_ep && (p.ep.steps & B200FC_STEP_QUANT) && p.ep.q_per_oc;
        const bool any_vec = use_deq || use_bias || use_q;
        int it = 0;
        bool ok = true;
        const unsigned leader_acc_empty = mapa_rank(bar_acc_empty, 0);
        for (int item = pair; item < num_items && ok; item += num_pairs, it++) {
            const int tile = item % num_tiles, split = item / num_tiles;
            const long long c_offset = (long long)split * p.split_stride;
            const int ab = it & 1;
            const unsigned acc_phase = (unsigned)(it >> 1) & 1;
            int tm, tn;
            tile_coords(p, tile, tm, tn);
            // while the tile's MMAs run: this warp's copy of the per-column vectors of the tile's BN columns (clamped
            // to the last valid column), so that no chunk waits for global memory
            if (any_vec) {
                const int nb = p.n0 + tn * BN;
#pragma unroll
                for (int j = 0; j < BN / 32; j++) {
                    const int col = min(nb + j * 32 + lane, p.n1 - 1);
                    if (use_deq) colvec[j * 32 + lane] = __ldg(p.ep.deq_per_oc + col);
                    if (use_bias) colvec[BN + j * 32 + lane] = __ldg(p.ep.bias + col);
                    if (use_q) colvec[2 * BN + j * 32 + lane] = __ldg(p.ep.q_per_oc + col);
                }
                __syncwarp();
            }
            if (!mbar_wait<EPI_SLEEP_NS>(bar_acc_full + 8 * ab, acc_phase, abort_flag, p.wait_limit_ns)) { ok = false; break; }
            tc_fence_after();
            const int m = tm * (2 * BM) + (int)rank * BM + quarter * 32 + lane;
            const bool row_ok = m < p.M;
            const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(ab * BN);
#pragma unroll 1
            for (int c = 0; c < BN / 32; c++) {
                const int n = p.n0 + tn * BN + c * 32;
                if (n >= p.n1) break;
                unsigned r[32];
                tc_ld32(taddr + (unsigned)(c * 32), r);
                tc_wait_ld();
                EpiArgs ea{&p.ep, p.vec_ok, p.acc_is_int, p.n1, p.M, epi_tile};
                if (use_deq) ea.cv_deq = colvec + c * 32;
                if (use_bias) ea.cv_bias = colvec + BN + c * 32;
                if (use_q) ea.cv_q = colvec + 2 * BN + c * 32;
                epilogue_chunk(r, m, n, ea, row_ok, c_offset);
            }
            tc_fence_before();
            if (p.ar_world) __threadfence_system();  // this warp's part of the tile is visible to every GPU ...
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_remote(leader_acc_empty + 8 * ab);
                if (p.ar_world)                      // ... before the tile's owner counts the arrival
                    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.ar_flags[tile % p.ar_world] + 2 * tile + (int)rank), "r"(1u)
                                 : "memory");
            }
        }
    }

    if (p.ar_world && !comm_role && p.ar_phases == 3) {
        // this CTA's tiles are done: help with the reduction of the tiles this rank owns (the last round's arrive late)
        __syncthreads();
        if (!*abort_flag) allreduce_units<BN>(p, num_tiles, unit_slot, abort_flag);
    }

    // ---------------- common exit ----------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            atomicExch(p.status, 2);
            const unsigned long long t0 = globaltimer();
            while (globaltimer() - t0 < 200000ull) { }
        }
        __syncthreads();
    }
    cluster_sync_all();  // the peer may still be signalling this CTA's barriers until here
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)C::TMEM_COLS)
                     : "memory");
    }
}

// ---- split-K reduction + post-ops ------------------------------------------------------------------------------------
// ws holds `splits` slabs of raw accumulators ([M][pitch], column index = global n - n0).  Each thread sums one output
// element over the slabs in slab order (deterministic) and runs the ordinary post-ops / SiLU pairing on it.
__global__ void splitk_reduce_kernel(const unsigned* __restrict__ ws, long long slab_elems, int pitch, int splits, int M,
                                     int n0, int n1, int acc_is_int, const Epilogue ep) {
    const bool silu = (ep.steps & B200FC_STEP_SILU_MUL) != 0;
    const int cols = silu ? (n1 - n0) / 2 : (n1 - n0);
    const long long total = (long long)M * cols;
    // launched as a programmatic dependent of the GEMM: resident early, waits here for the slabs
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // fp32 accumulators, four consecutive columns per thread: one 16-byte load per slab, all of them in flight together
    // (the scalar loop below is bound by the latency of its dependent 4-byte loads)
    if (!silu && !acc_is_int && !ep.residual && (cols & 3) == 0 && (pitch & 3) == 0 && splits <= 8 &&
        (ep.out_dtype == B200FC_F32 || ep.out_dtype == B200FC_BF16) && ((uintptr_t)ep.C & 15) == 0 && (ep.ldc & 15) == 0 &&
        (n0 & 3) == 0) {
        const int c4 = cols >> 2;
        const long long total4 = (long long)M * c4;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (long long)gridDim.x * blockDim.x) {
            const int m = (int)(i / c4), c = (int)(i % c4) * 4;
            const float4* src = (const float4*)(ws + (long long)m * pitch + c);
            float4 v[8];
#pragma unroll
            for (int q = 0; q < 8; q++)
                if (q < splits) v[q] = src[(long long)q * (slab_elems >> 2)];
            float4 sum = v[0];
#pragma unroll
            for (int q = 1; q < 8; q++)
                if (q < splits) { sum.x += v[q].x; sum.y += v[q].y; sum.z += v[q].z; sum.w += v[q].w; }
            const int n = n0 + c;
            const float o0 = postop_scalar(sum.x, n, ep), o1 = postop_scalar(sum.y, n + 1, ep);
            const float o2 = postop_scalar(sum.z, n + 2, ep), o3 = postop_scalar(sum.w, n + 3, ep);
            char* crow = (char*)ep.C + (long long)m * ep.ldc;
            if (ep.out_dtype == B200FC_F32) {
                *(float4*)(crow + (long long)n * 4) = make_float4(o0, o1, o2, o3);
            } else {
                const unsigned lo = (unsigned)f32_to_bf16_bits(o0) | ((unsigned)f32_to_bf16_bits(o1) << 16);
                const unsigned hi = (unsigned)f32_to_bf16_bits(o2) | ((unsigned)f32_to_bf16_bits(o3) << 16);
                *(uint2*)(crow + (long long)n * 2) = make_uint2(lo, hi);
            }
        }
        return;
    }
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int m = (int)(i / cols), c = (int)(i % cols);
        const unsigned* row = ws + (long long)m * pitch;
        if (silu) {
            const int gcol = 32 * (c >> 4) + (c & 15);
            float gsum = 0.0f, usum = 0.0f;
            for (int q = 0; q < splits; q++) {
                gsum += __uint_as_float(row[q * slab_elems + gcol]);
                usum += __uint_as_float(row[q * slab_elems + gcol + 16]);
            }
            unsigned short* crow = (unsigned short*)((char*)ep.C + (long long)m * ep.ldc);
            crow[(n0 >> 1) + c] = f32_to_bf16_bits(silu_f(gsum) * usum);
        } else if (acc_is_int) {
            int sum = 0;
            for (int q = 0; q < splits; q++) sum += (int)row[q * slab_elems + c];
            if (ep.out_dtype == B200FC_S32) ((int*)((char*)ep.C + (long long)m * ep.ldc))[n0 + c] = sum;
            else store_scalar(postop_scalar((float)sum, n0 + c, ep), m, n0 + c, ep);
        } else {
            float sum = 0.0f;
            for (int q = 0; q < splits; q++) sum += __uint_as_float(row[q * slab_elems + c]);
            store_scalar(postop_scalar(sum, n0 + c, ep), m, n0 + c, ep);
        }
    }
}

// ---- host side -----------------------------------------------------------------------------------------------------------
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

// 2-D K-major tensor map: inner dimension = K elements, outer = rows; box = {128 bytes of K, box_rows}.
int make_map(CUtensorMap* map, const void* base, bool i8, uint64_t k_elems, uint64_t rows, uint64_t ld_bytes,
             uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled entry point not available"); return B200FC_ERR_CUDA; }
    cuuint64_t dims[2] = {k_elems, rows};
    cuuint64_t strides[1] = {ld_bytes};
    cuuint32_t box[2] = {(cuuint32_t)(i8 ? SLAB_BYTES : SLAB_BYTES / 2), box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, i8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d)", (int)r); return B200FC_ERR_CUDA; }
    return B200FC_OK;
}

// tcgen05 instruction descriptor (dense, K-major A and B, M = 128): accumulator format bits [4,6), A format [7,10),
// B format [10,13), N >> 3 at [17,23), M >> 4 at [24,29).
unsigned make_idesc(bool i8, bool a_signed, bool b_signed, int bn, int mma_m = BM) {
    unsigned d = 0;
    if (i8) {
        d |= 2u << 4;                       // int32 accumulator
        d |= (a_signed ? 1u : 0u) << 7;     // 8-bit integer: 1 = signed, 0 = unsigned
        d |= (b_signed ? 1u : 0u) << 10;
    } else {
        d |= 1u << 4;                       // fp32 accumulator
        d |= 1u << 7;                       // bf16
        d |= 1u << 10;
    }
    d |= (unsigned)(bn >> 3) << 17;
    d |= (unsigned)(mma_m >> 4) << 24;
    return d;
}

int num_sms() {
    static std::atomic<int> cache[64];   // SM count per device ordinal (0 = not asked yet)
    int dev = 0;
    cudaGetDevice(&dev);
    int n = cache[dev & 63].load(std::memory_order_relaxed);
    if (!n) {
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
        cache[dev & 63].store(n, std::memory_order_relaxed);
    }
    // the persistent GEMM grids take one CTA per SM; a caller that overlaps a collective with them leaves it a few SMs
    const int lim = sm_limit();
    return (lim >= 2 && lim < n) ? (lim & ~1) : n;
}

template <int BN, bool I8>
int launch_cfg(const CUtensorMap& ma, const CUtensorMap& mw, const GemmParams& p, cudaStream_t s) {
    using C = Cfg<BN>;
    static std::atomic<unsigned long long> attr_devices{0};
    {
        const int arc = once_per_device(attr_devices, [] {
            B200FC_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN, I8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             C::SMEM_BYTES));
            return (int)B200FC_OK;
        });
        if (arc) return arc;
    }
    int tiles = p.tiles_m * p.tiles_n;
    int grid = tiles < num_sms() ? tiles : num_sms();
    gemm_tc_kernel<BN, I8><<<grid, NUM_THREADS, C::SMEM_BYTES, s>>>(ma, mw, p);
    count_launch();
    B200FC_CUDA(cudaGetLastError());
    return B200FC_OK;
}

template <int BN, bool I8>
int launch_cfg2(const CUtensorMap& ma, const CUtensorMap& mw, GemmParams p, cudaStream_t s) {
    using C = Cfg2<BN>;
    static std::atomic<unsigned long long> attr_devices{0};
    {
        const int arc = once_per_device(attr_devices, [] {
            B200FC_CUDA(cudaFuncSetAttribute(gemm_tc2_kernel<BN, I8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             C::SMEM_BYTES));
            return (int)B200FC_OK;
        });
        if (arc) return arc;
    }
    const int tiles = p.tiles_m * p.tiles_n;
    const int max_pairs = num_sms() / 2;
    // Too few tiles to occupy the GPU (small M): split K so that every pair has work; the raw partial accumulators go
    // through a workspace of this stream and a second kernel sums them in order and runs the post-ops.
    int splits = 1;
    if (tiles * 2 <= max_pairs && p.k_slabs >= 16 && !p.ep.mc_reduce) {
        splits = max_pairs / tiles;
        if (splits > 8) splits = 8;
        if (splits > p.k_slabs / 8) splits = p.k_slabs / 8;
        if (splits < 1) splits = 1;
    }
    p.splits = splits;
    p.split_stride = 0;
    const Epilogue final_ep = p.ep;
    const int final_vec = p.vec_ok;
    int pitch = 0;
    if (splits > 1) {
        const int nspan = p.n1 - p.n0;
        pitch = (nspan + 3) / 4 * 4;
        const size_t slab = (size_t)p.M * pitch * 4;
        void* ws = nullptr;
        int rc = get_stream_scratch(slab * splits, s, 1, &ws);
        if (rc) return rc;
        p.split_stride = (long long)slab;
        p.ep.steps = 0;
        p.ep.residual = nullptr;                    // (the reduction kernel adds it, with the caller's post-ops)
        p.ep.out_dtype = I8 ? B200FC_S32 : B200FC_F32;
        p.ep.C = (char*)ws - (long long)p.n0 * 4;   // the kernel indexes columns by the global n
        p.ep.ldc = (long long)pitch * 4;
        p.vec_ok = (p.n0 % 4) == 0 ? 1 : 0;
    }
    if (splits > 1) p.item_limit = 0;
    int items = p.item_limit > 0 ? p.item_limit : tiles * splits;
    int pairs = items < max_pairs ? items : max_pairs;
    gemm_tc2_kernel<BN, I8><<<2 * pairs, NUM_THREADS, C::SMEM_BYTES, s>>>(ma, mw, p);
    count_launch();
    B200FC_CUDA(cudaGetLastError());
    if (splits > 1) {
        const long long total = (long long)p.M * (p.n1 - p.n0);
        long long blocks = (total + 255) / 256;
        if (blocks > 148 * 8) blocks = 148 * 8;
        // programmatic dependent launch: the reduction's blocks become resident while the GEMM drains (the GEMM
        // triggers its dependents at its start) and wait inside the kernel, which hides the launch latency
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)blocks, 1, 1);
        cfg.blockDim = dim3(256, 1, 1);
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        B200FC_CUDA(cudaLaunchKernelEx(&cfg, splitk_reduce_kernel, (const unsigned*)((char*)p.ep.C + (long long)p.n0 * 4),
                                       (long long)p.M * pitch, pitch, splits, p.M, p.n0, p.n1, p.acc_is_int, final_ep));
        count_launch();
    }
    (void)final_vec;
    return B200FC_OK;
}

// B200FC_GEMM_PANEL=n: row tiles per panel of the 2-CTA GEMM's tile order (0 = no panels); unset = by shape
int panel_rows_setting() {
    static int v = -2;
    if (v == -2) {
        const char* e = getenv("B200FC_GEMM_PANEL");
        v = e ? atoi(e) : -1;
    }
    return v;
}

// B200FC_GEMM_TAIL=0 keeps the tiles of a ragged last round in the main launch (for measurements)
bool tail_split_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("B200FC_GEMM_TAIL");
        v = e ? atoi(e) : 1;
    }
    return v != 0;
}

// 0 = choose by shape, 1 = force the 1-CTA kernel, 2 = force the 2-CTA kernel (B200FC_GEMM_CTAS, for experiments)
int forced_ctas() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("B200FC_GEMM_CTAS");
        v = e ? atoi(e) : 0;
    }
    return v;
}

}  // namespace

int launch_gemm_tc_allreduce(const void* W_data, int W_K_pad, int W_N_pad, const void* A, int M, int K, int64_t lda,
                             int N, const AllReduceDesc& ar, cudaStream_t s) {
    if (((uintptr_t)A & 15) || (lda & 15)) { set_error("gemm allreduce: A must be 16-byte aligned"); return B200FC_ERR_INVALID; }
    if (ar.world < 2 || ar.world > 8 || ar.rank < 0 || ar.rank >= ar.world) { set_error("gemm allreduce: bad rank / world"); return B200FC_ERR_INVALID; }
    if ((N & 7) || (ar.ld_bytes & 15) || ((uintptr_t)ar.partial_local & 15) || ((uintptr_t)ar.partial_mc & 15) || ((uintptr_t)ar.out_mc & 15)) {
        set_error("gemm allreduce: N must be a multiple of 8 and the buffers 16-byte aligned");
        return B200FC_ERR_INVALID;
    }
    if (M <= 0) return B200FC_OK;
    GemmParams p;
    p.M = M; p.K = K; p.n0 = 0; p.n1 = N;
    p.tiles_m = (M + 2 * BM - 1) / (2 * BM);
    p.tiles_n = (N + 255) / 256;
    if (2 * p.tiles_m * p.tiles_n > ar.max_tiles - 1) { set_error("gemm allreduce: %d arrival counters needed, %d given", 2 * p.tiles_m * p.tiles_n, ar.max_tiles); return B200FC_ERR_INVALID; }
    p.k_slabs = (K + 63) / 64;
    p.idesc = make_idesc(false, false, false, 256, 2 * BM);
    p.acc_is_int = 0;
    p.ep.steps = 0; p.ep.out_dtype = B200FC_BF16; p.ep.C = ar.partial_local; p.ep.ldc = ar.ld_bytes;
    p.ep.bias = nullptr; p.ep.deq_scale = 1.0f; p.ep.deq_per_oc = nullptr; p.ep.q_scale = 1.0f; p.ep.q_per_oc = nullptr;
    p.ep.mc_reduce = 0;
    p.vec_ok = 1;
    p.status = kernel_status_word();
    if (!p.status) { set_error("gemm: no kernel status word on this device"); return B200FC_ERR_CUDA; }
    p.wait_limit_ns = wait_limit_ns();
    p.splits = 1; p.split_stride = 0;
    p.ar_world = ar.world; p.ar_rank = ar.rank;
    {
        const char* e = getenv("B200FC_AR_PHASES");
        p.ar_phases = e ? atoi(e) : 3;
    }
    const int all_pairs = num_sms() / 2;
    int comm_pairs = ar.comm_sms / 2;
    if (comm_pairs < 1) comm_pairs = 1;
    if (comm_pairs > all_pairs - 1) comm_pairs = all_pairs - 1;
    p.ar_gemm_pairs = all_pairs - comm_pairs;
    p.ar_target = (unsigned)ar.world * 4u;
    p.ar_work_counter = ar.max_tiles - 1;
    for (int i = 0; i < 8; i++) p.ar_flags[i] = i < ar.world ? ar.flags[i] : nullptr;
    p.ar_partial_mc = (const char*)ar.partial_mc;
    p.ar_out_mc = (char*)ar.out_mc;
    CUtensorMap ma, mw;
    int rc = make_map(&ma, A, false, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BM);
    if (rc) return rc;
    rc = make_map(&mw, W_data, false, (uint64_t)W_K_pad, (uint64_t)W_N_pad, (uint64_t)W_K_pad * 2, 128);
    if (rc) return rc;
    using C = Cfg2<256>;
    static std::atomic<unsigned long long> attr_devices{0};
    {
        const int arc = once_per_device(attr_devices, [] {
            B200FC_CUDA(cudaFuncSetAttribute(gemm_tc2_kernel<256, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
            return (int)B200FC_OK;
        });
        if (arc) return arc;
    }
    // the whole grid must be resident (reducing pairs wait for multiplying pairs of every GPU): one CTA per SM
    gemm_tc2_kernel<256, false><<<2 * all_pairs, NUM_THREADS, C::SMEM_BYTES, s>>>(ma, mw, p);
    count_launch();
    B200FC_CUDA(cudaGetLastError());
    return B200FC_OK;
}

int launch_gemm_tc(const void* W_data, int w_dtype, int W_K_pad, int W_N_pad, const void* A, int dtypeA, int M, int K,
                   int64_t lda, int n0, int n1, const Epilogue& ep, cudaStream_t s) {
    const bool i8 = dtypeA != B200FC_BF16;
    if (i8 != (w_dtype != B200FC_BF16)) { set_error("gemm_tc: activation / weight dtype mismatch"); return B200FC_ERR_INVALID; }
    if (((uintptr_t)A & 15) || (lda & 15)) {
        set_error("gemm_tc: A must be 16-byte aligned with a 16-byte multiple leading dimension");
        return B200FC_ERR_INVALID;
    }
    if (M <= 0 || n1 <= n0) return B200FC_OK;
    const int nspan = n1 - n0;
    // 256-wide tiles unless that leaves SMs idle while 128-wide tiles would not
    const int tiles_m = (M + BM - 1) / BM;
    int bn = 256;
    {
        int t256 = tiles_m * ((nspan + 255) / 256), t128 = tiles_m * ((nspan + 127) / 128);
        int sms = num_sms();
        auto waves_eff = [&](int t) { return (double)t / (double)(((t + sms - 1) / sms) * sms); };
        if (nspan <= 128 || (t256 < sms && t128 > t256) || waves_eff(t128) > waves_eff(t256) + 0.08) bn = 128;
    }
    GemmParams p;
    p.M = M; p.K = K; p.n0 = n0; p.n1 = n1;
    p.tiles_m = tiles_m;
    p.tiles_n = (nspan + bn - 1) / bn;
    const int slab_elems = i8 ? SLAB_BYTES : SLAB_BYTES / 2;
    p.k_slabs = (K + slab_elems - 1) / slab_elems;
    p.idesc = make_idesc(i8, dtypeA == B200FC_S8, w_dtype == B200FC_S8, bn);
    p.acc_is_int = i8 ? 1 : 0;
    p.ep = ep;
    p.status = kernel_status_word();
    if (!p.status) { set_error("gemm: no kernel status word on this device"); return B200FC_ERR_CUDA; }
    p.wait_limit_ns = wait_limit_ns();
    p.splits = 1; p.split_stride = 0;
    p.ar_world = 0; p.ar_rank = 0; p.ar_phases = 3; p.ar_gemm_pairs = 0; p.ar_work_counter = 0; p.ar_target = 0; p.ar_partial_mc = nullptr; p.ar_out_mc = nullptr;
    for (int i = 0; i < 8; i++) p.ar_flags[i] = nullptr;
    int es = ep.out_dtype == B200FC_F32 || ep.out_dtype == B200FC_S32 ? 4 : (ep.out_dtype == B200FC_BF16 ? 2 : 1);
    if (ep.steps & B200FC_STEP_SILU_MUL)
        p.vec_ok = (((uintptr_t)ep.C & 15) == 0 && (ep.ldc & 15) == 0 && (n0 % 32) == 0) ? 1 : 0;
    else
        p.vec_ok = (((uintptr_t)ep.C & 15) == 0 && (ep.ldc & 15) == 0 && ((n0 * es) & 15) == 0) ? 1 : 0;
    if (ep.out_dtype == B200FC_S32 && !i8) { set_error("raw int32 output needs an 8-bit GEMM"); return B200FC_ERR_INVALID; }
    if (ep.mc_reduce && (ep.steps != 0 || i8 || ((n0 | n1) & 1) || ((uintptr_t)ep.C & 3) || (ep.ldc & 3))) {
        set_error("multicast-reduce output needs a bf16 GEMM without post-ops and an even, 4-byte aligned column range");
        return B200FC_ERR_INVALID;
    }

    CUtensorMap ma, mw;
    int rc = make_map(&ma, A, i8, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BM);
    if (rc) return rc;
    // 2-CTA tiles (256 x 256 per CTA pair) when there are at least two 128-row blocks of M and enough tiles
    // ... or when the 1-CTA kernel would leave most SMs without a tile while K is long (the 2-CTA launcher splits K)
    const bool few_tiles = tiles_m * ((nspan + 255) / 256) * 2 <= num_sms() / 2 && K >= 2048;
    const bool pair_ok = (forced_ctas() == 2) || (forced_ctas() == 0 && nspan > 128 && (M > BM || few_tiles));
    if (pair_ok) {
        const int bn2 = 256;
        p.tiles_m = (M + 2 * BM - 1) / (2 * BM);
        p.tiles_n = (nspan + bn2 - 1) / bn2;
        p.idesc = make_idesc(i8, dtypeA == B200FC_S8, w_dtype == B200FC_S8, bn2, 2 * BM);
        rc = make_map(&mw, W_data, i8, (uint64_t)W_K_pad, (uint64_t)W_N_pad, (uint64_t)W_K_pad * (i8 ? 1 : 2),
                      (uint32_t)(bn2 / 2));
        if (rc) return rc;
        // Ragged last round: tiles % pairs tiles would occupy a few CTA pairs for a whole tile time while the others
        // idle (Llama-70B gate/up at M = 1024: 896 tiles on 74 pairs, 8 left over).  When the tile time is long (K >=
        // 6144) and the left-over tiles (the last ones in tile order) form one rectangle — whole column blocks, or the
        // bottom of the last one — the main launch stops before them and they go through this function again as a
        // GEMM of their own, which takes the K-split route (a few tiles, every pair busy for a fraction of a tile
        // time, then the reduction kernel with the same post-ops).
        const int tiles = p.tiles_m * p.tiles_n, pairs = num_sms() / 2;
        // Activations larger than what stays in L2 beside the streaming weights (the whole of them is touched by every
        // round of tiles): take the tiles panel by panel so that only panel_rows x 256 rows are live at a time, and keep
        // those in L2 (evict-last hint on their loads).  Weights are then read once per panel.
        {
            const int want = panel_rows_setting();
            const size_t a_bytes = (size_t)M * (size_t)K * (i8 ? 1 : 2);
            if (want > 0) p.panel_rows = want;
            else if (want < 0 && a_bytes > ((size_t)48 << 20) && p.tiles_m >= 12 && p.tiles_n >= 2 * pairs / 8) p.panel_rows = 8;
            if (p.panel_rows >= p.tiles_m) p.panel_rows = 0;
        }
        const int rem = tiles % pairs;
        const int last_cols = nspan - (p.tiles_n - 1) * bn2;
        // (the last tiles in tile order lie in the last panel, ph row tiles high)
        const int ph = p.panel_rows > 0 ? p.tiles_m - (p.tiles_m - 1) / p.panel_rows * p.panel_rows : p.tiles_m;
        const int whole = rem / ph, part = rem % ph;   // whole column blocks of that panel / tiles of a partial one
        if (tail_split_enabled() && tiles > pairs && rem > 0 && (whole == 0 || part == 0) && rem * 4 <= pairs &&
            p.k_slabs >= 96 && last_cols > 128 && !ep.mc_reduce) {
            p.item_limit = tiles - rem;
            rc = i8 ? launch_cfg2<256, true>(ma, mw, p, s) : launch_cfg2<256, false>(ma, mw, p, s);
            if (rc) return rc;
            const long long row0 = (long long)(p.tiles_m - (whole ? ph : part)) * 2 * BM;
            const int col0 = n0 + (p.tiles_n - (whole ? whole : 1)) * bn2;
            Epilogue e2 = ep;
            e2.C = (char*)ep.C + row0 * ep.ldc;
            if (ep.residual) e2.residual = (const char*)ep.residual + row0 * ep.ld_res;
            return launch_gemm_tc(W_data, w_dtype, W_K_pad, W_N_pad, (const char*)A + row0 * lda, dtypeA, (int)(M - row0), K, lda,
                                  col0, n1, e2, s);
        }
        return i8 ? launch_cfg2<256, true>(ma, mw, p, s) : launch_cfg2<256, false>(ma, mw, p, s);
    }
    rc = make_map(&mw, W_data, i8, (uint64_t)W_K_pad, (uint64_t)W_N_pad, (uint64_t)W_K_pad * (i8 ? 1 : 2), (uint32_t)bn);
    if (rc) return rc;
    if (bn == 256) return i8 ? launch_cfg<256, true>(ma, mw, p, s) : launch_cfg<256, false>(ma, mw, p, s);
    return i8 ? launch_cfg<128, true>(ma, mw, p, s) : launch_cfg<128, false>(ma, mw, p, s);
}

}  // namespace b200fc
