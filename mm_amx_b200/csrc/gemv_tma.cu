// Decode-shaped fully-connected layer (M <= 16 rows of bf16 activations): an HBM-bound weight stream.
//
// Replaces the M <= 16 branches of amx_kernel::Matmul (include/kernels_amx.hpp:1216-1253), of the compressed-weight
// specialisation Matmul<bf16,int8_t,float> (kernels_amx.hpp:1381-1441) and its stand-alone development version
// matmul16m_Wint8B (weight_compression/fc16m.cpp:451-502), plus the M <= 16 case of the fused MLP
// (tests/amx-mlp.cpp:707-737, 648-704).
//
// How the bytes move
//   The packed weights are [N_pad, K_pad] with K contiguous.  The unit of the stream is a 16 KB stage: 128 weight rows
//   x 128 bytes of K, one 2-D TMA box with 128-byte swizzle.  All stages of the call — row blocks outermost, K inside —
//   form one sequence that is cut into equal contiguous pieces, one per CTA ("stream-K"), so every SM streams the
//   same number of bytes whatever N and K are.  One producer warp per CTA keeps a ring of 4-5 stages in flight; eight
//   consumer warps copy their share of a stage (32 rows x 64 bytes of K) into registers (conflict-free through the
//   swizzle), release the stage and feed mma.sync.m16n8k16 with the weights as the 16-row operand and the <= 16
//   activation rows as the 8-column operand (K permuted identically on both sides, which a dot product does not see).
//   Compressed (int8) weights are stored offset-binary (v + 128): one byte permute builds the fp16 number
//   1024 + v + 128, one subtraction leaves v — one instruction per weight, next to the consumer (the role of the
//   reference's ping-pong dequantisation buffer).  fp16 because only its 11-bit significand holds all 8 bits; the
//   activations are converted to fp16 per staged chunk after an exact power-of-two scaling per row.
//   4-bit weights (two values per byte, a stage holds 256 K of 128 rows = two quantisation groups): masks and one shift
//   per word build the fp16 numbers 1024 + n and 1024 + 16 n of the nibbles n = v + 8, a subtraction resp. a fused
//   multiply-add leaves v.  The packing keeps the four lanes of an MMA inside one group, so every stage is multiplied
//   into a fresh accumulator that is added to the running one times the group's fp32 scale (integer-valued partial
//   sums: the scale is applied once per group, exactly as the definition of the format says).  The stage's 2 x 128
//   scales travel beside it (one 1 KB bulk copy on the same barrier).
//   A piece that ends inside a row block leaves a partial sum: it goes to a slot of a small global scratch, the CTAs
//   that share the row block count themselves on a counter, and the last one to arrive adds the slots in CTA order
//   (deterministic) and runs the post-ops.  Nobody waits for anybody.
//   The grid is at most one CTA per SM although two fit: with programmatic dependent launch the next kernel of the
//   stream becomes resident beside this one and fills its own ring while this one still computes, so a chain of
//   decode layers keeps HBM busy across kernel boundaries (weights never depend on the previous kernel; activations,
//   the scratch and the output are touched only after griddepcontrol.wait).
//   full[s]  : TMA complete_tx + one arrive.expect_tx by the producer        empty[s] : one arrive per consumer warp
// All mbarrier waits are bounded; on a time-out the CTA raises an abort flag, every role stops waiting, the kernel
// stores an error code and still publishes (meaningless) partial sums so that the counters return to zero.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cstdlib>
#include "common.cuh"

namespace b200fc {

namespace {

constexpr int CWARPS = 8;                       // consumer warps
constexpr int CTHREADS = CWARPS * 32;
constexpr int ROWS_PER_WARP = 32;               // a warp owns 32 rows x one 64-byte half of every stage
constexpr int ROWS_PER_CTA = (CWARPS / 2) * ROWS_PER_WARP;  // 128
constexpr int STAGE_K_BYTES = 128;              // bytes of K per row and stage (one swizzle atom)
constexpr int STAGE_BYTES = ROWS_PER_CTA * STAGE_K_BYTES;  // 16 KB
constexpr int THREADS = (CWARPS + 1) * 32;
constexpr int SLOT_FLOATS = 16 * ROWS_PER_CTA;  // one partial-sum slot: [16 activation rows][128 weight rows] fp32

struct Params {
    int spr;              // stages per packed row (K_pad bytes / 128)
    long long total;      // stages of the whole call: row blocks x spr
    int S;                // > 0: every row block is cut into S pieces, CTA c takes piece c % S of row block c / S;
                          // 0: the whole stage sequence is cut into gridDim.x equal pieces ("stream-K")
    const unsigned char* X;
    long long ldx;
    int M, K;
    int n0, n1;
    Epilogue ep;
    int* status;
    float* slots;         // [gridDim.x][2][SLOT_FLOATS]: partial sums of the first / last piece of each CTA
    unsigned* counters;   // [gridDim.x], zero between launches
    unsigned long long wait_limit_ns;
    int cluster;          // 1: launched as clusters of S CTAs (S <= 8); the pieces of a row block meet in distributed
                          // shared memory instead of the global scratch
    int pf_cap;           // stages beyond the ring that the producer prefetches into L2 when the CTA starts
    const float* scales;  // 4-bit weights: [row block][stage][2][128] group scales, row block 0 = packed rows [0, 128)
    const unsigned char* ximg;   // quantised weights, optional: the activations already converted by xstage_kernel, one
                                 // image of the shared-memory chunk buffer per CHUNK of K ([chunk][MP][XROW], the row's
                                 // exponent in the first word of its pad); null = the consumers convert them themselves
#ifdef B200FC_TRACE
    unsigned long long* trace;   // [launch % 64][gridDim.x <= 320][8] globaltimer stamps (timeline studies only)
    int trace_launch;
#endif
};

#ifdef B200FC_TRACE
#define TRACE_STAMP(i) do { if (p.trace && (threadIdx.x & 31) == 0) p.trace[((size_t)(p.trace_launch & 63) * 320 + blockIdx.x) * 8 + (i)] = globaltimer(); } while (0)
#else
#define TRACE_STAMP(i) do { } while (0)
#endif

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
// Bounded wait.  try_wait itself suspends the thread for a while, so the loop is not hot; the clock and the abort flag
// are looked at only after a batch of failed attempts (reading %globaltimer is slow, and doing it after every failed
// attempt delayed the moment a consumer notices its stage by that much).
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag, unsigned long long limit) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = 0;
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 16; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        const unsigned long long now = globaltimer();
        if (t0 == 0) t0 = now;
        if (now - t0 > limit) {
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
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// fp32 at shared-memory address `addr` (of this CTA's window) in CTA `rank` of the cluster
__device__ __forceinline__ float ld_peer_f32(unsigned addr, unsigned rank) {
    unsigned ra;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
    return v;
}
// strong (coherent at GPU scope) 16-byte load: partial sums written by other SMs during this launch
__device__ __forceinline__ float4 ld_gpu_f4(const float4* p) {
    float4 v;
    asm volatile("ld.relaxed.gpu.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory"); }

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
// two offset-binary weights (bytes `sel` of w) -> f16x2 holding their values exactly:
// 0x64xx is the fp16 number 1024 + xx, and 1024 + (v + 128) - 1152 = v
__device__ __forceinline__ unsigned u8x2_to_f16x2(unsigned w, unsigned sel) {
    unsigned p = __byte_perm(w, 0x64646464u, sel);
    const __half2 off = __floats2half2_rn(1152.0f, 1152.0f);
    __half2 r = __hsub2(*(__half2*)&p, off);
    return *(unsigned*)&r;
}

__device__ __forceinline__ void cp_async16(unsigned dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void bulk_load_1d(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// (w & mask) | 0x64006400: the two nibbles selected by `mask` as the low bits of two fp16 numbers 1024 + ...
__device__ __forceinline__ unsigned nib_or_magic(unsigned w, unsigned mask) {
    unsigned r;
    asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(r) : "r"(w), "r"(mask), "r"(0x64006400u));   // (a & b) | c
    return r;
}
// nibbles n at bits [0,4) and [16,20) of w -> f16x2 of n - 8:  (1024 + n) - 1032
__device__ __forceinline__ unsigned nib_lo_to_f16x2(unsigned w) {
    const unsigned p = nib_or_magic(w, 0x000f000fu), off = 0x64086408u;   // 1032.0 twice
    __half2 r = __hsub2(*(const __half2*)&p, *(const __half2*)&off);
    return *(unsigned*)&r;
}
// nibbles n at bits [4,8) and [20,24) of w -> f16x2 of n - 8:  (1024 + 16 n) / 16 - 72
__device__ __forceinline__ unsigned nib_hi_to_f16x2(unsigned w) {
    const unsigned p = nib_or_magic(w, 0x00f000f0u), mul = 0x2c002c00u, add = 0xd480d480u;   // 1/16 and -72 twice
    __half2 r = __hfma2(*(const __half2*)&p, *(const __half2*)&mul, *(const __half2*)&add);
    return *(unsigned*)&r;
}

// acc * 2^d for |d| <= 252 as two multiplications by exact powers of two (scalbnf costs ~20 instructions per value and
// the accumulators change their scale at most chunk boundaries)
__device__ __forceinline__ void pow2_factors(int d, float& f1, float& f2) {
    d = d < -252 ? -252 : (d > 252 ? 252 : d);
    const int h = d / 2;
    f1 = __int_as_float((127 + h) << 23);
    f2 = __int_as_float((127 + d - h) << 23);
}

template <int WB, int NT> struct Layout {
    static constexpr bool WQ = WB != 16;   // quantised weights: activations are staged as fp16
    static constexpr int STAGES = (NT == 1 && !WQ) ? 5 : 4;
    static constexpr int MP = 8 * NT;
    // activation elements staged per chunk; quantised weights keep a second, raw copy of the NEXT chunk (see RAW_OFF)
    static constexpr int CHUNK = (WQ && NT == 2) ? 512 : 1024;
    // bytes per staged activation row; the pad makes rows g and g + 1 fall into different bank halves for the
    // access pattern of each variant (see the fragment loads in the kernel)
    static constexpr int XROW = CHUNK * 2 + (WQ ? 64 : 16);
    static constexpr int RING = STAGES * STAGE_BYTES;
    static constexpr int X_OFF = RING;
    static constexpr int AUX_OFF = X_OFF + MP * XROW;          // smax [MP][CWARPS], sexp [MP]
    static constexpr int EP_OFF = AUX_OFF + MP * (CWARPS + 1) * 4;   // dequant scale, bias, quant scale of 128 rows
    static constexpr int SC_OFF = EP_OFF + 3 * ROWS_PER_CTA * 4;     // 4-bit weights: group scales of every ring stage
    static constexpr int SC_STAGE_BYTES = 2 * ROWS_PER_CTA * 4;
    // quantised weights: the next chunk's activations as they lie in global memory (bf16), fetched with cp.async while
    // the current chunk is multiplied; every thread copies, reads back and overwrites only its own 16-byte units
    static constexpr int RAW_OFF = SC_OFF + (WB == 4 ? STAGES * SC_STAGE_BYTES : 0);
    // (with pre-converted activations the same region is the second chunk buffer, filled while the first is in use)
    static constexpr int BAR_OFF = RAW_OFF + (WQ ? MP * XROW : 0);
    static constexpr int SMEM = BAR_OFF + 2 * STAGES * 8 + 16 + 1024;  // + barriers, abort flag, last flag, alignment slack
};

// first stage of CTA c's piece, and the CTA whose piece holds stage s
__device__ __forceinline__ long long piece_begin(const Params& p, int G, int c) {
    if (p.S > 0) return (long long)(c / p.S) * p.spr + (long long)p.spr * (c % p.S) / p.S;
    return p.total * c / G;      // pieces are [c * total / G, (c + 1) * total / G)
}
__device__ __forceinline__ int piece_of(const Params& p, int G, long long s) {
    if (p.S > 0) {
        const int rb = (int)(s / p.spr), ks = (int)(s - (long long)rb * p.spr);
        return rb * p.S + (int)((((long long)ks + 1) * p.S - 1) / p.spr);
    }
    return (int)(((s + 1) * G - 1) / p.total);
}

// DEQUANT -> BIAS -> GELU -> QUANT on one value of weight row `row` of the current row block; s_ep holds the three
// per-row vectors (dequant scale, bias, quant scale), loaded next to the activations so that the epilogue does not
// wait for global memory again
__device__ __forceinline__ float postop_staged(float v, int row, int steps, const float* s_ep) {
    if (steps & B200FC_STEP_DEQUANT) v *= s_ep[row];
    if (steps & B200FC_STEP_BIAS) v += s_ep[ROWS_PER_CTA + row];
    if (steps & B200FC_STEP_GELU) v = gelu_erf_poly(v);
    if (steps & B200FC_STEP_QUANT) v *= s_ep[2 * ROWS_PER_CTA + row];
    return v;
}

// The kernel body.  NJ = 1: one matrix.  NJ = 2: two dependent matrices in ONE launch (the decode-shaped MLP: gate/up with
// the SiLU*up store, then the down projection over the activation the first job wrote): the producer goes straight on
// into the second matrix, so its first ring of stages arrives while the consumers finish the first job and wait at a
// grid-wide barrier (every CTA must have stored its part of the activation before anyone multiplies by it).
template <int WB, int NT, int NJ>
__device__ __forceinline__ void decode_body(const CUtensorMap* map0, const CUtensorMap* map1, const Params* p0, const Params* p1) {
    const Params& p = *p0;            // job 0; the role loops below shadow it with the job they work on
    using L = Layout<WB, NT>;
    constexpr bool W8 = WB == 8, W4 = WB == 4, WQ = WB != 16;
    constexpr int MP = L::MP, XROW = L::XROW, STAGES = L::STAGES;
    constexpr int KE = STAGE_K_BYTES * 8 / WB;        // K elements per stage: 64 / 128 / 256
    constexpr int CHUNK_K = L::CHUNK;
    constexpr int STAGES_PER_CHUNK = CHUNK_K / KE;
    constexpr int MMA_PER_LOAD = 32 / WB;             // MMAs (16 K each) fed by one 16-byte piece of two rows

    extern __shared__ unsigned char smem_raw[];
    // aligned to 1024 bytes by pointer arithmetic on the __shared__ array itself: through an integer round trip the
    // compiler loses the address space and every access below becomes a generic load / store (slower, 64-bit addresses)
    unsigned char* smem = smem_raw + (((smem_u32(smem_raw) + 1023u) & ~1023u) - smem_u32(smem_raw));
    unsigned char* xbuf = smem + L::X_OFF;
    unsigned char* xcur = xbuf;   // chunk buffer the MMAs read: xbuf, or with pre-converted activations xbuf / the raw region in turn
    unsigned* smax = (unsigned*)(smem + L::AUX_OFF);
    int* sexp = (int*)(smem + L::AUX_OFF + MP * CWARPS * 4);
    const unsigned bar_full = smem_u32(smem + L::BAR_OFF);
    const unsigned bar_empty = bar_full + STAGES * 8;
    volatile int* abort_flag = (volatile int*)(smem + L::BAR_OFF + 2 * STAGES * 8);
    volatile int* last_flag = abort_flag + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int G = (int)gridDim.x, cta = (int)blockIdx.x;
    const unsigned long long limit = p.wait_limit_ns;

    if (threadIdx.x == 0) {
        TRACE_STAMP(0);   // CTA started
        asm volatile("prefetch.tensormap [%0];" ::"l"(map0) : "memory");
        if (NJ > 1) asm volatile("prefetch.tensormap [%0];" ::"l"(map1) : "memory");
        for (int i = 0; i < STAGES; i++) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, CWARPS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // the next kernel in the stream may become resident and start its own weight stream now
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == CWARPS) {
        // ---------------- producer: weights never depend on the previous kernel, stream at once ----------------
        if (lane == 0) {
            int stage = 0;
            unsigned phase = 0;
            bool alive = true;
#pragma unroll 1
            for (int job = 0; job < NJ && alive; job++) {
            const Params& p = job ? *p1 : *p0;
            const CUtensorMap* map_w = job ? map1 : map0;
            const long long it_begin = piece_begin(p, G, cta), it_end = piece_begin(p, G, cta + 1);
            int rb = (int)(it_begin / p.spr), ks = (int)(it_begin - (long long)rb * p.spr);
            for (long long it = it_begin; it < it_end; it++) {
                if (it == it_begin + STAGES && p.pf_cap > 0) {
                    // The ring is full and this CTA may have to wait for the previous kernel of the stream: ask L2
                    // for the next stages meanwhile, so that their DRAM round trip is not paid later, one ring slot
                    // at a time, on the path between two dependent kernels.
                    long long pf_to = it + p.pf_cap < it_end ? it + p.pf_cap : it_end;
                    int pf_rb = rb, pf_ks = ks;
                    for (long long pf = it; pf < pf_to; pf++) {
                        tma_prefetch_l2_2d(map_w, pf_ks * STAGE_K_BYTES, p.n0 + pf_rb * ROWS_PER_CTA);
                        if (++pf_ks == p.spr) { pf_ks = 0; pf_rb++; }
                    }
                }
                if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, limit)) { alive = false; break; }
                mbar_expect_tx(bar_full + 8 * stage, STAGE_BYTES + (W4 ? L::SC_STAGE_BYTES : 0));
                tma_load_2d(smem_u32(smem + stage * STAGE_BYTES), map_w, bar_full + 8 * stage, ks * STAGE_K_BYTES,
                            p.n0 + rb * ROWS_PER_CTA);
                if constexpr (W4)
                    bulk_load_1d(smem_u32(smem + L::SC_OFF + stage * L::SC_STAGE_BYTES),
                                 p.scales + ((size_t)(p.n0 / ROWS_PER_CTA + rb) * p.spr + ks) * (2 * ROWS_PER_CTA),
                                 L::SC_STAGE_BYTES, bar_full + 8 * stage);
                if (++ks == p.spr) { ks = 0; rb++; }
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
            }
        }
    } else {
        // ---------------- consumers ----------------
        // activations, the scratch and the output may belong to the previous kernel of the stream until here
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (threadIdx.x == 0) TRACE_STAMP(1);   // previous kernel complete
        const int ctid = threadIdx.x;                        // 0 .. 255
        int stage = 0;
        unsigned phase = 0;
        bool ok = true;
#pragma unroll 1
        for (int job = 0; job < NJ; job++) {
        const Params& p = job ? *p1 : *p0;
        const long long it_begin = piece_begin(p, G, cta), it_end = piece_begin(p, G, cta + 1);
        xcur = xbuf;
        const bool x_vec = (((uintptr_t)p.X & 15) == 0) && ((p.ldx & 15) == 0);
        const bool x_fast = x_vec && (p.K & 7) == 0;
        auto load_x_unit = [&](int row, int k) -> uint4 {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (x_fast) {
                // no branch around the load, so that the loads of all passes are in flight together: out-of-range
                // units read element (0, 0) and are zeroed afterwards
                const bool in = row < p.M && k < p.K;
                const uint4 r = *(const uint4*)(p.X + (long long)(in ? row : 0) * p.ldx + (long long)(in ? k : 0) * 2);
                return in ? r : v;
            }
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
        constexpr int RB = ROWS_PER_WARP / 16;  // 16-row MMA blocks per warp
        // AS > 1 would give every MMA of a 16-byte weight load its own accumulator set (shorter dependent chains);
        // measured slower (the extra registers spill), so one set is used.
        constexpr int AS = 1;
        float acc[AS][RB][NT][4];
        // Compressed weights multiply fp16 x fp16, so every staged chunk is scaled per activation row by the power of two
        // that puts the row's largest magnitude (within the chunk) at 2^13 and converted to fp16: exact, since fp16 keeps
        // the 8-bit significand of bf16.  The accumulators carry the row's current scale (cur_e) and are rescaled when a
        // new chunk brings a different one; the scale is undone after the last stage of a piece.
        int cur_e[NT][2];

        // Stages CHUNK_K activation elements of all MP rows, starting at stage ks of a row: UNITS sixteen-byte units per
        // row, the 256 consumer threads take ROWS_PER_PASS rows per pass.  All loads of a thread are issued before the
        // first is converted / stored.
        constexpr int UNITS = CHUNK_K / 8;                    // 128 or 64
        constexpr int ROWS_PER_PASS = CTHREADS / UNITS;       // 2 or 4
        constexpr int PASSES = MP / ROWS_PER_PASS;
        constexpr int WPR = UNITS / 32;                       // consumer warps that share one activation row
        const int unit = ctid % UNITS, row0 = ctid / UNITS;
        unsigned char* xraw = smem + L::RAW_OFF;
        // Quantised weights: asks for the chunk that starts at stage ks (this thread's units of it) to be copied into the
        // raw buffer.  Called for the first chunk of a piece right before it is staged, and for every later chunk right
        // after the previous one has been staged, so that the copy runs under a whole chunk of multiplications: the
        // global-memory latency of the activations (about a microsecond while the weight stream saturates the memory
        // system) otherwise stops all eight warps at every chunk boundary.
        auto prefetch_x = [&](int ks, int ks_end) {
            if constexpr (WQ) {
                if (x_fast) {
                    const int k = ks * KE + unit * 8;
                    if (k < ks_end * KE && k < p.K) {
#pragma unroll
                        for (int i = 0; i < PASSES; i++) {
                            const int row = row0 + i * ROWS_PER_PASS;
                            if (row < p.M)
                                cp_async16(smem_u32(xraw + (row * UNITS + unit) * 16), p.X + (long long)row * p.ldx + (long long)k * 2);
                        }
                    }
                    asm volatile("cp.async.commit_group;" ::: "memory");
                }
            }
        };
        auto stage_x = [&](int ks, int ks_end, bool more) {
            const int k = ks * KE + unit * 8;
            const bool need = k < ks_end * KE;
            const bool raw = WQ && x_fast;
            // bf16 weights store right after the loads: everyone must be done with the previous chunk first.  The raw path
            // stores only after the barrier that follows the maximum search, which no warp reaches before it has finished
            // the previous chunk.
            if (!raw) consumer_sync();
            if (threadIdx.x == 0 && ks * KE < CHUNK_K) TRACE_STAMP(6);   // staging of a first chunk begins
            uint4 v[PASSES];
            if (raw) {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
                for (int i = 0; i < PASSES; i++) {
                    const int row = row0 + i * ROWS_PER_PASS;
                    v[i] = (need && row < p.M && k < p.K) ? *(const uint4*)(xraw + (row * UNITS + unit) * 16) : make_uint4(0, 0, 0, 0);
                }
            } else {
#pragma unroll
                for (int i = 0; i < PASSES; i++) v[i] = need ? load_x_unit(row0 + i * ROWS_PER_PASS, k) : make_uint4(0, 0, 0, 0);
            }
            if constexpr (WQ) {
#pragma unroll
                for (int i = 0; i < PASSES; i++) {
                    const unsigned w4[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
                    unsigned m = 0;
#pragma unroll
                    for (int q = 0; q < 4; q++) m = max(m, max(w4[q] & 0x7fffu, (w4[q] >> 16) & 0x7fffu));
                    m = __reduce_max_sync(0xffffffffu, m);
                    if (lane == 0) smax[(row0 + i * ROWS_PER_PASS) * CWARPS + warp] = m;   // WPR of the 8 slots per row
                }
                consumer_sync();
                // the raw values are in registers: the same units may now receive the next chunk
                if (more) prefetch_x(ks + STAGES_PER_CHUNK, ks_end);
            }
#pragma unroll
            for (int i = 0; i < PASSES; i++) {
                const int row = row0 + i * ROWS_PER_PASS;
                uint4 o4 = v[i];
                if constexpr (WQ) {
                    // the warps that hold this row: warps WPR * row0 .. WPR * row0 + WPR - 1
                    unsigned m = 0;
#pragma unroll
                    for (int q = 0; q < WPR; q++) m = max(m, smax[row * CWARPS + row0 * WPR + q]);
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
                // int8 weights: the 16 units of a stage are stored transposed as a 4 x 4 grid, so that the four lanes t
                // of a fragment load (units 4t + i) touch four neighbouring 16-byte slots; 4-bit weights: the 32 units
                // of a stage as a 4 x 8 grid (a lane reads units 4 (4h + t) + i, i = 0..3)
                const int slot = W8 ? ((unit & ~15) | ((unit & 3) << 2) | ((unit >> 2) & 3))
                               : W4 ? ((unit & ~31) | ((unit & 3) << 3) | ((unit >> 2) & 7)) : unit;
                if (need) *(uint4*)(xbuf + row * XROW + slot * 16) = o4;
            }
            consumer_sync();
            if constexpr (WQ) {
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const int e0 = sexp[nt * 8 + 2 * t], e1 = sexp[nt * 8 + 2 * t + 1];
                    if (cur_e[nt][0] != e0 || cur_e[nt][1] != e1) {
                        float a1, a2, b1, b2;
                        pow2_factors(cur_e[nt][0] - e0, a1, a2);
                        pow2_factors(cur_e[nt][1] - e1, b1, b2);
#pragma unroll
                        for (int as = 0; as < AS; as++)
#pragma unroll
                            for (int rb = 0; rb < RB; rb++) {
                                acc[as][rb][nt][0] = acc[as][rb][nt][0] * a1 * a2;
                                acc[as][rb][nt][2] = acc[as][rb][nt][2] * a1 * a2;
                                acc[as][rb][nt][1] = acc[as][rb][nt][1] * b1 * b2;
                                acc[as][rb][nt][3] = acc[as][rb][nt][3] * b1 * b2;
                            }
                        cur_e[nt][0] = e0; cur_e[nt][1] = e1;
                    }
                }
            }
        };

        // Pre-converted activations (p.ximg): the chunk images lie ready in global memory (L2), chunk c covering stages
        // [c * STAGES_PER_CHUNK, +STAGES_PER_CHUNK) of every row whatever piece reads them.  A chunk boundary is then one
        // wait for the copy issued a chunk earlier and ONE barrier; nothing is converted here.
        const bool img = WQ && p.ximg != nullptr;
        int xb = 0;
        constexpr int IMG_BYTES = MP * XROW;
        auto copy_img = [&](int c, int buf) {
            const unsigned char* src = p.ximg + (size_t)c * IMG_BYTES;
            const unsigned dst = smem_u32(buf ? xraw : xbuf);
            for (int u = ctid; u < IMG_BYTES / 16; u += CTHREADS) cp_async16(dst + u * 16, src + u * 16);
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        auto stage_img = [&](int ks, int ks0, int ks_end, bool first_piece) {
            if constexpr (WQ) {
                const int c = ks / STAGES_PER_CHUNK;
                if (ks == ks0) {
                    // a piece's first chunk: nothing is in flight.  The previous piece's partial tile lies over xbuf and
                    // may still be read by a slower warp.
                    if (!first_piece) consumer_sync();
                    copy_img(c, xb);
                }
                asm volatile("cp.async.wait_group 0;" ::: "memory");
                consumer_sync();   // every thread's part of the image is there; every warp has left the previous chunk
                if ((c + 1) * STAGES_PER_CHUNK < ks_end) copy_img(c + 1, xb ^ 1);
                xcur = xb ? xraw : xbuf;
                xb ^= 1;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const int e0 = *(const int*)(xcur + (nt * 8 + 2 * t) * XROW + CHUNK_K * 2);
                    const int e1 = *(const int*)(xcur + (nt * 8 + 2 * t + 1) * XROW + CHUNK_K * 2);
                    if (cur_e[nt][0] != e0 || cur_e[nt][1] != e1) {
                        float a1, a2, b1, b2;
                        pow2_factors(cur_e[nt][0] - e0, a1, a2);
                        pow2_factors(cur_e[nt][1] - e1, b1, b2);
#pragma unroll
                        for (int rb = 0; rb < RB; rb++) {
                            acc[0][rb][nt][0] = acc[0][rb][nt][0] * a1 * a2;
                            acc[0][rb][nt][2] = acc[0][rb][nt][2] * a1 * a2;
                            acc[0][rb][nt][1] = acc[0][rb][nt][1] * b1 * b2;
                            acc[0][rb][nt][3] = acc[0][rb][nt][3] * b1 * b2;
                        }
                        cur_e[nt][0] = e0; cur_e[nt][1] = e1;
                    }
                }
            }
        };

        // byte offsets of this thread's 16-byte pieces inside a stage: rows (rb, h) -> warp*32 + rb*16 + h*8 + g,
        // logical chunk 2t + j, physical chunk = logical ^ (row & 7) = logical ^ g
        const int rg = warp >> 1, kh = warp & 1;       // row group (32 rows) and K half (64 bytes) of this warp
        const int row_base = rg * ROWS_PER_WARP + g;
        float* part = (float*)xbuf;                    // partial tiles of a finished piece: part[K half][token][row]
        constexpr int PART_HALF = MP * ROWS_PER_CTA;   // floats per K half
        const Epilogue& ep = p.ep;
        const bool silu = (ep.steps & B200FC_STEP_SILU_MUL) != 0;
        float* s_ep = (float*)(smem + L::EP_OFF);

        long long it = it_begin;
        while (it < it_end) {
            // ---- one piece: stages [ks0, ks1) of row block rbk ----
            const int rbk = (int)(it / p.spr);
            const int ks0 = (int)(it - (long long)rbk * p.spr);
            const int ks1 = (long long)(p.spr - ks0) < it_end - it ? p.spr : ks0 + (int)(it_end - it);
            const bool first_piece = it == it_begin;
#pragma unroll
            for (int as = 0; as < AS; as++)
#pragma unroll
                for (int rb = 0; rb < RB; rb++)
#pragma unroll
                    for (int nt = 0; nt < NT; nt++)
#pragma unroll
                        for (int i = 0; i < 4; i++) acc[as][rb][nt][i] = 0.0f;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) cur_e[nt][0] = cur_e[nt][1] = 0;

            // post-op vectors of this row block (one row per thread of the first four warps); the loads travel together
            // with those of the first activation chunk
            float ep_deq = 1.0f, ep_bias = 0.0f, ep_q = 1.0f;
            if (ctid < ROWS_PER_CTA) {
                const int n = p.n0 + rbk * ROWS_PER_CTA + ctid;
                if (n < p.n1) {
                    if (ep.steps & B200FC_STEP_DEQUANT) ep_deq = ep.deq_per_oc ? ep.deq_scale * ep.deq_per_oc[n] : ep.deq_scale;
                    if (ep.steps & B200FC_STEP_BIAS) ep_bias = ep.bias[n];
                    if (ep.steps & B200FC_STEP_QUANT) ep_q = ep.q_per_oc ? ep.q_per_oc[n] : ep.q_scale;
                }
            }
            for (int ks = ks0; ks < ks1; ks++) {
                const int it_in_chunk = img ? ks % STAGES_PER_CHUNK : (ks - ks0) % STAGES_PER_CHUNK;
                if (it_in_chunk == 0 || ks == ks0) {
                    if (img) {
                        stage_img(ks, ks0, ks1, first_piece);
                    } else {
                        if (ks == ks0) prefetch_x(ks, ks1);                   // nothing was in flight for a piece's first chunk
                        stage_x(ks, ks1, ks + STAGES_PER_CHUNK < ks1);
                    }
                }
                if (ks == ks0 && ctid < ROWS_PER_CTA) {
                    // (the first barrier of stage_x has been passed: nobody still reads the previous piece's vectors)
                    s_ep[ctid] = ep_deq; s_ep[ROWS_PER_CTA + ctid] = ep_bias; s_ep[2 * ROWS_PER_CTA + ctid] = ep_q;
                }
                if (threadIdx.x == 0 && ks == ks0 && first_piece) TRACE_STAMP(2);   // first activation chunk staged
                // warp-uniform outcome: either every lane goes on to the MMAs or none does
                ok = __all_sync(0xffffffffu, ok && mbar_wait(bar_full + 8 * stage, phase, abort_flag, limit));
                if (threadIdx.x == 0 && ks == ks0 && first_piece) TRACE_STAMP(7);   // first stage of weights is there
                if (!ok) continue;
                uint4 w[RB][2];
                const unsigned char* sbase = smem + stage * STAGE_BYTES;
#pragma unroll
                for (int rb = 0; rb < RB; rb++)
#pragma unroll
                    for (int h = 0; h < 2; h++)
                        w[rb][h] = *(const uint4*)(sbase + (row_base + rb * 16 + h * 8) * STAGE_K_BYTES + (((2 * t + kh) ^ g) << 4));
                const int rel_stage = stage;
                if (++stage == STAGES) { stage = 0; phase ^= 1; }

                const int j = kh;
                if constexpr (W4) {
                    // this thread's 32 K of the stage, [128 j + 32 t, +32) — all of group j — sit in four slots 128 bytes apart
                    const int xoff = it_in_chunk * KE * 2 + (4 * j + t) * 16;
                    unsigned xb[NT][16];
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        const unsigned char* xs = xcur + (nt * 8 + g) * XROW + xoff;
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const uint4 a = *(const uint4*)(xs + i * 128);
                            xb[nt][4 * i] = a.x; xb[nt][4 * i + 1] = a.y; xb[nt][4 * i + 2] = a.z; xb[nt][4 * i + 3] = a.w;
                        }
                    }
                    const float* sc = (const float*)(smem + L::SC_OFF + rel_stage * L::SC_STAGE_BYTES) + j * ROWS_PER_CTA + row_base;
#pragma unroll
                    for (int rb = 0; rb < RB; rb++) {
                        const unsigned wa[4] = {w[rb][0].x, w[rb][0].y, w[rb][0].z, w[rb][0].w};
                        const unsigned wb[4] = {w[rb][1].x, w[rb][1].y, w[rb][1].z, w[rb][1].w};
                        float grp[NT][4];
#pragma unroll
                        for (int nt = 0; nt < NT; nt++)
#pragma unroll
                            for (int c = 0; c < 4; c++) grp[nt][c] = 0.0f;
#pragma unroll
                        for (int i = 0; i < 4; i++) {
#pragma unroll
                            for (int hw = 0; hw < 2; hw++) {        // values 0..3 and 4..7 of word i
                                const unsigned qa = wa[i] >> (8 * hw), qb = wb[i] >> (8 * hw);
                                const unsigned a0 = nib_lo_to_f16x2(qa), a2 = nib_hi_to_f16x2(qa);
                                const unsigned a1 = nib_lo_to_f16x2(qb), a3 = nib_hi_to_f16x2(qb);
#pragma unroll
                                for (int nt = 0; nt < NT; nt++)
                                    mma_f16(grp[nt], a0, a1, a2, a3, xb[nt][4 * i + 2 * hw], xb[nt][4 * i + 2 * hw + 1]);
                            }
                        }
                        const float s0 = sc[rb * 16], s1 = sc[rb * 16 + 8];
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) {
                            acc[0][rb][nt][0] = fmaf(grp[nt][0], s0, acc[0][rb][nt][0]);
                            acc[0][rb][nt][1] = fmaf(grp[nt][1], s0, acc[0][rb][nt][1]);
                            acc[0][rb][nt][2] = fmaf(grp[nt][2], s1, acc[0][rb][nt][2]);
                            acc[0][rb][nt][3] = fmaf(grp[nt][3], s1, acc[0][rb][nt][3]);
                        }
                    }
                } else {
                // activations matching this thread's weight bytes: K elements [(2t + j) * (W8 ? 16 : 8), ...) of the stage
                const int xoff = W8 ? it_in_chunk * KE * 2 + (8 * j + t) * 16 : (it_in_chunk * KE + (2 * t + j) * 8) * 2;
                unsigned xb[NT][W8 ? 8 : 4];
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const unsigned char* xs = xcur + (nt * 8 + g) * XROW + xoff;
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
                            if constexpr (W8) mma_f16(acc[q % AS][rb][nt], a0, a1, a2, a3, xb[nt][2 * q], xb[nt][2 * q + 1]);
                            else mma_bf16(acc[q % AS][rb][nt], a0, a1, a2, a3, xb[nt][2 * q], xb[nt][2 * q + 1]);
                        }
                    }
                }
                }
                // Release the stage only now that its bytes have gone through the MMAs.  Arriving right after the copies to
                // registers had been issued (or even after folding them into a dummy value) let the refill overtake them
                // now and then: single rows of a warp's share then held bytes of the stage four positions later.
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_empty + 8 * rel_stage);
            }
            it += ks1 - ks0;
            if (threadIdx.x == 0 && it == it_end) TRACE_STAMP(3);   // last stage multiplied
            // the accumulator sets are added in a fixed order
#pragma unroll
            for (int as = 1; as < AS; as++)
#pragma unroll
                for (int rb = 0; rb < RB; rb++)
#pragma unroll
                    for (int nt = 0; nt < NT; nt++)
#pragma unroll
                        for (int i = 0; i < 4; i++) acc[0][rb][nt][i] += acc[as][rb][nt][i];
            if constexpr (WQ) {
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                    for (int rb = 0; rb < RB; rb++) {
                        acc[0][rb][nt][0] = scalbnf(acc[0][rb][nt][0], cur_e[nt][0]);
                        acc[0][rb][nt][2] = scalbnf(acc[0][rb][nt][2], cur_e[nt][0]);
                        acc[0][rb][nt][1] = scalbnf(acc[0][rb][nt][1], cur_e[nt][1]);
                        acc[0][rb][nt][3] = scalbnf(acc[0][rb][nt][3], cur_e[nt][1]);
                    }
            }

            // ---- the piece's partial tile -> shared memory (over the activation buffer) ----
            consumer_sync();
#pragma unroll
            for (int rb = 0; rb < RB; rb++)
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const int row = rg * ROWS_PER_WARP + rb * 16 + g, tok = nt * 8 + 2 * t;
                    float* pp = part + kh * PART_HALF;
                    pp[tok * ROWS_PER_CTA + row] = acc[0][rb][nt][0];
                    pp[(tok + 1) * ROWS_PER_CTA + row] = acc[0][rb][nt][1];
                    pp[tok * ROWS_PER_CTA + row + 8] = acc[0][rb][nt][2];
                    pp[(tok + 1) * ROWS_PER_CTA + row + 8] = acc[0][rb][nt][3];
                }
            consumer_sync();

            // ---- who finishes the row block?  a piece that covers it alone does; otherwise the last CTA to arrive ----
            const bool whole = ks0 == 0 && ks1 == p.spr;
            int c_first = cta, c_last = cta;
            bool finish = true;
            if (p.cluster) {
                // the two K halves are added here; the cluster's CTAs then share the rest of the work (end of kernel)
                for (int e = ctid; e < p.M * ROWS_PER_CTA; e += CTHREADS) part[e] += part[PART_HALF + e];
                finish = false;
            } else if (!whole) {
                const int nvec = p.M * ROWS_PER_CTA / 4;
                float4* slot = (float4*)(p.slots + (size_t)(2 * cta + (first_piece ? 0 : 1)) * SLOT_FLOATS);
                for (int v = ctid; v < nvec; v += CTHREADS) {
                    const float4 a = ((const float4*)part)[v], b = ((const float4*)(part + PART_HALF))[v];
                    slot[v] = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
                }
                // every writer fences its own stores: a release by thread 0 alone (after the barrier) was observed NOT to
                // cover the other warps' stores — now and then a reader summed a slot before all of it had arrived
                __threadfence();
                consumer_sync();
                const long long s_first = (long long)rbk * p.spr;
                c_first = piece_of(p, G, s_first);
                c_last = piece_of(p, G, s_first + p.spr - 1);
                if (ctid == 0) {
                    // release: the slot stores of all consumer threads (ordered before this by the barrier) are visible to
                    // whoever reads the counter; acquire: so are the slots of the CTAs that counted themselves earlier
                    unsigned old;
                    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(p.counters + c_first) : "memory");
                    const bool last = old == (unsigned)(c_last - c_first);
                    if (last) p.counters[c_first] = 0;   // the counter is ready for the next launch
                    *last_flag = last ? 1 : 0;
                }
                consumer_sync();
                if (threadIdx.x == 0 && it == it_end) TRACE_STAMP(4);   // counted
                finish = *last_flag != 0;
                if (finish) {
                    // Sum the slots of the CTAs that share the row block, in CTA order, into part[token][row].  Only the
                    // first of them can hold the row block as the piece that CLOSES its range (slot 1); for all others it
                    // opens their range (slot 0).  Eight slots are read at a time so that the L2 round trips overlap.
                    // every reader fences too: thread 0's acquire alone does not cover the other warps' loads
                    __threadfence();
                    const int which_first = piece_begin(p, G, c_first) < s_first ? 1 : 0;
                    const float4* base = (const float4*)p.slots;
                    for (int v = ctid; v < nvec; v += CTHREADS) {
                        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        for (int c = c_first; c <= c_last; c += 8) {
                            float4 t4[8];
#pragma unroll
                            for (int u = 0; u < 8; u++) {
                                const int cc = c + u;
                                const int which = cc == c_first ? which_first : 0;
                                t4[u] = cc <= c_last ? ld_gpu_f4(base + (size_t)(2 * cc + which) * (SLOT_FLOATS / 4) + v)
                                                     : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                            }
#pragma unroll
                            for (int u = 0; u < 8; u++) {
                                sum.x += t4[u].x; sum.y += t4[u].y; sum.z += t4[u].z; sum.w += t4[u].w;
                            }
                        }
                        ((float4*)part)[v] = sum;
                    }
                    consumer_sync();
                }
            }
            if (finish) {
                // value of element [token][row] of the row block
                auto reduced = [&](int idx) -> float { return whole ? part[idx] + part[PART_HALF + idx] : part[idx]; };
                const int blk_row0 = p.n0 + rbk * ROWS_PER_CTA;
                const int out_rows = silu ? ROWS_PER_CTA / 2 : ROWS_PER_CTA;
                const int n_out = out_rows * p.M;
                for (int e = ctid; e < n_out; e += CTHREADS) {
                    const int tok = e / out_rows, orow = e % out_rows;
                    if (silu) {
                        const int grow = 32 * (orow >> 4) + (orow & 15);
                        if (blk_row0 + grow + 16 < p.n1) {
                            const float gsum = reduced(tok * ROWS_PER_CTA + grow), usum = reduced(tok * ROWS_PER_CTA + grow + 16);
                            unsigned short* crow = (unsigned short*)((char*)ep.C + (long long)tok * ep.ldc);
                            crow[(blk_row0 >> 1) + orow] = f32_to_bf16_bits(silu_f(gsum) * usum);
                        }
                    } else {
                        const int n = blk_row0 + orow;
                        if (n < p.n1) store_scalar(postop_staged(reduced(tok * ROWS_PER_CTA + orow), orow, ep.steps, s_ep), tok, n, ep);
                    }
                }
            }
        }
        if constexpr (NJ > 1) {
            // ---- between two jobs: every CTA's stores of the first job (the activation) must be visible before any CTA
            // reads them.  Arrivals are counted on a word of the scratch; the wait is bounded like every other one. ----
            unsigned* gbar = p.counters + (kGemvMaxCtas - 2);     // [0] arrivals, [1] CTAs that finished the launch
            if (job + 1 < NJ) {
                __threadfence();          // every writer fences its own stores (see the slot exchange above)
                consumer_sync();
                if (ctid == 0) {
                    unsigned seen;
                    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(seen) : "l"(gbar) : "memory");
                    seen += 1;
                    unsigned long long t0 = 0;
                    while (seen < (unsigned)G && !*abort_flag) {
                        __nanosleep(100);     // 296 pollers on one word would otherwise delay the arrivals themselves
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(gbar) : "memory");
                        if (seen >= (unsigned)G) break;
                        const unsigned long long now = globaltimer();
                        if (t0 == 0) t0 = now;
                        if (now - t0 > limit) *abort_flag = 1;
                    }
                }
                consumer_sync();
                __threadfence();          // every reader fences too
                if (*abort_flag) ok = false;
            } else if (ctid == 0) {
                // the launch's last CTA to get here leaves both words zero for the next launch
                unsigned done;
                asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(done) : "l"(gbar + 1) : "memory");
                if (done == (unsigned)(G - 1)) { gbar[0] = 0; gbar[1] = 0; }
            }
        }
        }   // jobs
        if (ctid == 0) TRACE_STAMP(5);   // done
    }

    if (NJ == 1 && p.cluster) {
        // ---- the S pieces of this row block meet: every CTA of the cluster finishes 1/S of the outputs, adding the
        // partial tiles of all S CTAs in rank order (deterministic) ----
        __syncwarp();
        cluster_sync_all();
        if (threadIdx.x == 0) TRACE_STAMP(4);   // all pieces of the row block are there
        const int S = p.S, rank = cta % S, blk_row0 = p.n0 + (cta / S) * ROWS_PER_CTA;
        const unsigned part_addr = smem_u32(xbuf);
        const Epilogue& ep = p.ep;
        const bool silu = (ep.steps & B200FC_STEP_SILU_MUL) != 0;
        const int out_rows = silu ? ROWS_PER_CTA / 2 : ROWS_PER_CTA;
        const int n_out = out_rows * p.M;
        const int e_begin = (int)((long long)n_out * rank / S), e_end = (int)((long long)n_out * (rank + 1) / S);
        const float* s_ep = (const float*)(smem + L::EP_OFF);
        for (int e = e_begin + (int)threadIdx.x; e < e_end; e += THREADS) {
            const int tok = e / out_rows, orow = e % out_rows;
            if (silu) {
                const int grow = 32 * (orow >> 4) + (orow & 15);
                float gsum = 0.0f, usum = 0.0f;
                for (int q = 0; q < S; q++) {
                    gsum += ld_peer_f32(part_addr + 4u * (unsigned)(tok * ROWS_PER_CTA + grow), (unsigned)q);
                    usum += ld_peer_f32(part_addr + 4u * (unsigned)(tok * ROWS_PER_CTA + grow + 16), (unsigned)q);
                }
                if (blk_row0 + grow + 16 < p.n1) {
                    unsigned short* crow = (unsigned short*)((char*)ep.C + (long long)tok * ep.ldc);
                    crow[(blk_row0 >> 1) + orow] = f32_to_bf16_bits(silu_f(gsum) * usum);
                }
            } else {
                float sum = 0.0f;
                for (int q = 0; q < S; q++) sum += ld_peer_f32(part_addr + 4u * (unsigned)(tok * ROWS_PER_CTA + orow), (unsigned)q);
                const int n = blk_row0 + orow;
                if (n < p.n1) store_scalar(postop_staged(sum, orow, ep.steps, s_ep), tok, n, ep);
            }
        }
        if (threadIdx.x == 0) TRACE_STAMP(5);
        cluster_sync_all();  // nobody leaves while a peer may still read its partial tile
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, 3);
}

template <int WB, int NT>
__global__ void __launch_bounds__(THREADS, 2) gemv_tma_kernel(const __grid_constant__ CUtensorMap map_w, const Params p) {
    decode_body<WB, NT, 1>(&map_w, &map_w, &p, &p);
}

// gate/up (SiLU*up store into the activation) and down projection of a decode-shaped MLP in one launch (bf16 weights)
template <int NT>
__global__ void __launch_bounds__(THREADS, 2) mlp_decode_kernel(const __grid_constant__ CUtensorMap map_gate_up,
                                                                const __grid_constant__ CUtensorMap map_down,
                                                                const Params p_gate_up, const Params p_down) {
    decode_body<16, NT, 2>(&map_gate_up, &map_down, &p_gate_up, &p_down);
}


// Converts the activations of a call with quantised weights ONCE: block c writes the image of chunk c as the decode
// kernel's chunk buffer wants it — per row CHUNK fp16 values, scaled by the power of two that puts the row's largest
// magnitude within the chunk at 2^13 (exact: fp16 keeps the 8-bit significand of bf16), in the slot order of the
// variant's fragment loads, followed by a 64-byte pad whose first word is the exponent.  Rows >= M are zeros.  Used for
// large matrices, where every CTA walks several chunks and would otherwise convert them itself behind two CTA-wide
// barriers per chunk; the images (M_pad x K x 2 bytes) stay in L2.
template <int WB, int NT>
__global__ void __launch_bounds__(CTHREADS) xstage_kernel(const unsigned char* __restrict__ X, long long ldx, int M, int K,
                                                          unsigned char* __restrict__ img) {
    using L = Layout<WB, NT>;
    constexpr int MP = L::MP, XROW = L::XROW, CHUNK_K = L::CHUNK;
    constexpr int UNITS = CHUNK_K / 8, ROWS_PER_PASS = CTHREADS / UNITS, PASSES = MP / ROWS_PER_PASS, WPR = UNITS / 32;
    __shared__ unsigned smax[MP * CWARPS];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int ctid = threadIdx.x, warp = ctid >> 5, lane = ctid & 31;
    const int unit = ctid % UNITS, row0 = ctid / UNITS;
    const int k = blockIdx.x * CHUNK_K + unit * 8;
    const bool x_vec = (((uintptr_t)X & 15) == 0) && ((ldx & 15) == 0);
    uint4 v[PASSES];
#pragma unroll
    for (int i = 0; i < PASSES; i++) {
        const int row = row0 + i * ROWS_PER_PASS;
        v[i] = make_uint4(0, 0, 0, 0);
        if (row < M && k < K) {
            const unsigned char* src = X + (long long)row * ldx + (long long)k * 2;
            if (x_vec && k + 8 <= K) {
                v[i] = *(const uint4*)src;
            } else {
                unsigned short e[8];
#pragma unroll
                for (int q = 0; q < 8; q++) e[q] = (k + q < K) ? ((const unsigned short*)src)[q] : (unsigned short)0;
                v[i] = make_uint4(e[0] | ((unsigned)e[1] << 16), e[2] | ((unsigned)e[3] << 16), e[4] | ((unsigned)e[5] << 16),
                                  e[6] | ((unsigned)e[7] << 16));
            }
        }
    }
#pragma unroll
    for (int i = 0; i < PASSES; i++) {
        const unsigned w4[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
        unsigned m = 0;
#pragma unroll
        for (int q = 0; q < 4; q++) m = max(m, max(w4[q] & 0x7fffu, (w4[q] >> 16) & 0x7fffu));
        m = __reduce_max_sync(0xffffffffu, m);
        if (lane == 0) smax[(row0 + i * ROWS_PER_PASS) * CWARPS + warp] = m;
    }
    __syncthreads();
    unsigned char* out = img + (size_t)blockIdx.x * (MP * XROW);
#pragma unroll
    for (int i = 0; i < PASSES; i++) {
        const int row = row0 + i * ROWS_PER_PASS;
        unsigned m = 0;
#pragma unroll
        for (int q = 0; q < WPR; q++) m = max(m, smax[row * CWARPS + row0 * WPR + q]);
        int field = (int)(m >> 7);
        field = field < 1 ? 1 : field;
        int e = field - 127 - 13;
        e = e < -126 ? -126 : e;
        const float sc = __int_as_float((127 - e) << 23);
        const unsigned w4[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
        unsigned o[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            __half2 h = __floats2half2_rn(__uint_as_float(w4[q] << 16) * sc, __uint_as_float(w4[q] & 0xffff0000u) * sc);
            o[q] = *(unsigned*)&h;
        }
        const int slot = WB == 8 ? ((unit & ~15) | ((unit & 3) << 2) | ((unit >> 2) & 3))
                                 : ((unit & ~31) | ((unit & 3) << 3) | ((unit >> 2) & 7));
        *(uint4*)(out + row * XROW + slot * 16) = make_uint4(o[0], o[1], o[2], o[3]);
        if (unit < 4) *(uint4*)(out + row * XROW + CHUNK_K * 2 + unit * 16) = make_uint4(unit == 0 ? (unsigned)e : 0u, 0u, 0u, 0u);
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// The decode kernel on the 5th-generation tensor cores (bf16 weights, activations whose rows TMA can address).
// Same stream of 16 KB weight stages, same pieces, scratch exchange and post-ops as gemv_tma_kernel, but the products are
// tcgen05.mma instructions issued by one thread: A = the stage as TMA wrote it (128 weight rows x 64 K, K-major, 128-byte
// swizzle: the canonical operand layout), B = a 16-token x 64 K tile of the activations that travels with the stage
// (second TMA box, rows >= M zero-filled), D = 128 rows x 16 tokens of fp32 in TMEM.  No register copies of the
// weights, no activation staging, no barriers between the warps in the loop; sixteen tokens cost what one costs.
// Roles: warps 0-7 finish pieces (warps 0-3 read the accumulator, one TMEM lane quarter each), warp 8 lane 0 = TMA
// producer, warp 9 lane 0 = MMA issuer.  Two accumulator buffers (2 x 16 TMEM columns) let the issuer start the next
// piece while the previous one is reduced.
constexpr int TC_THREADS = (CWARPS + 2) * 32;
constexpr int TC_X_BYTES = 16 * STAGE_K_BYTES;             // activation tile of a stage: 16 tokens x 128 bytes of K
constexpr int TC_STAGE_BYTES = STAGE_BYTES + TC_X_BYTES;   // 18 KB, a multiple of 1024
constexpr int TC_STAGES = 5;
struct TcLayout {
    static constexpr int RING = TC_STAGES * TC_STAGE_BYTES;
    static constexpr int PART_OFF = RING;                              // [16 tokens][128 rows] fp32
    static constexpr int EP_OFF = PART_OFF + 16 * ROWS_PER_CTA * 4;
    static constexpr int BAR_OFF = EP_OFF + 3 * ROWS_PER_CTA * 4;      // full[S], empty[S], acc_full[2], acc_empty[2]
    static constexpr int SMEM = BAR_OFF + (2 * TC_STAGES + 4) * 8 + 32 + 1024;
};

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(unsigned d_tmem, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                            unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// K-major tile with rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart (descriptor version 1)
__device__ __forceinline__ unsigned long long tc_smem_desc(unsigned smem_addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)1 << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
__device__ __forceinline__ void tc_ld16(unsigned taddr, unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__global__ void __launch_bounds__(TC_THREADS, 2) gemv_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                const __grid_constant__ CUtensorMap map_x, const Params p) {
    using L = TcLayout;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + (((smem_u32(smem_raw) + 1023u) & ~1023u) - smem_u32(smem_raw));
    float* part = (float*)(smem + L::PART_OFF);
    float* s_ep = (float*)(smem + L::EP_OFF);
    const unsigned bar_full = smem_u32(smem + L::BAR_OFF);
    const unsigned bar_empty = bar_full + TC_STAGES * 8;
    const unsigned bar_acc_full = bar_empty + TC_STAGES * 8;
    const unsigned bar_acc_empty = bar_acc_full + 2 * 8;
    unsigned* tmem_holder = (unsigned*)(smem + L::BAR_OFF + (2 * TC_STAGES + 4) * 8);
    volatile int* abort_flag = (volatile int*)(tmem_holder + 1);
    volatile int* last_flag = abort_flag + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = (int)gridDim.x, cta = (int)blockIdx.x;
    const long long it_begin = piece_begin(p, G, cta), it_end = piece_begin(p, G, cta + 1);
    const unsigned long long limit = p.wait_limit_ns;

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        for (int i = 0; i < TC_STAGES; i++) {
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
    if (warp == CWARPS + 1) {   // the issuer's warp owns the tensor memory: 32 columns = two accumulators of 16
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(32u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const unsigned tmem_base = *tmem_holder;

    if (warp == CWARPS) {
        // ---------------- producer ----------------
        if (lane == 0) {
            int stage = 0;
            unsigned phase = 0;
            int rb = (int)(it_begin / p.spr), ks = (int)(it_begin - (long long)rb * p.spr);
            // weights never depend on the previous kernel: the first ring of stages is asked for at once, its activation
            // tiles only after the previous kernel of the stream has completed
            const long long n_first = it_end - it_begin < TC_STAGES ? it_end - it_begin : TC_STAGES;
            {
                int rb2 = rb, ks2 = ks;
                for (int i = 0; i < (int)n_first; i++) {
                    mbar_expect_tx(bar_full + 8 * i, TC_STAGE_BYTES);
                    tma_load_2d(smem_u32(smem + i * TC_STAGE_BYTES), &map_w, bar_full + 8 * i, ks2 * STAGE_K_BYTES, p.n0 + rb2 * ROWS_PER_CTA);
                    if (++ks2 == p.spr) { ks2 = 0; rb2++; }
                }
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            bool alive = true;
            for (long long it = it_begin; it < it_end && alive; it++) {
                const bool pre = it - it_begin < n_first;     // weights already on their way
                if (!pre) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, limit)) { alive = false; break; }
                    mbar_expect_tx(bar_full + 8 * stage, TC_STAGE_BYTES);
                    tma_load_2d(smem_u32(smem + stage * TC_STAGE_BYTES), &map_w, bar_full + 8 * stage, ks * STAGE_K_BYTES,
                                p.n0 + rb * ROWS_PER_CTA);
                }
                tma_load_2d(smem_u32(smem + stage * TC_STAGE_BYTES + STAGE_BYTES), &map_x, bar_full + 8 * stage, ks * (STAGE_K_BYTES / 2), 0);
                if (++ks == p.spr) { ks = 0; rb++; }
                if (++stage == TC_STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == CWARPS + 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // instruction descriptor: fp32 accumulator, bf16 x bf16, K-major operands, N = 16, M = 128
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
            int stage = 0;
            unsigned phase = 0;
            int piece = 0;
            bool alive = true;
            long long it = it_begin;
            while (it < it_end && alive) {
                const int rbk = (int)(it / p.spr);
                const int ks0 = (int)(it - (long long)rbk * p.spr);
                const int ks1 = (long long)(p.spr - ks0) < it_end - it ? p.spr : ks0 + (int)(it_end - it);
                const int ab = piece & 1;
                if (!mbar_wait(bar_acc_empty + 8 * ab, ((unsigned)(piece >> 1) & 1) ^ 1, abort_flag, limit)) { alive = false; break; }
                tc_fence_after();
                const unsigned d_tmem = tmem_base + (unsigned)(ab * 16);
                for (int ks = ks0; ks < ks1; ks++) {
                    if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, limit)) { alive = false; break; }
                    tc_fence_after();
                    const unsigned sa = smem_u32(smem + stage * TC_STAGE_BYTES);
                    const unsigned long long adesc = tc_smem_desc(sa), bdesc = tc_smem_desc(sa + STAGE_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; k++)     // 4 x 16 K per stage, 32 bytes further along the swizzled row each
                        tc_mma_bf16(d_tmem, adesc + (unsigned long long)(k * 2), bdesc + (unsigned long long)(k * 2), idesc,
                                    (unsigned)(((ks - ks0) | k) != 0));
                    tc_commit(bar_empty + 8 * stage);
                    if (ks == ks1 - 1) tc_commit(bar_acc_full + 8 * ab);
                    if (++stage == TC_STAGES) { stage = 0; phase ^= 1; }
                }
                it += ks1 - ks0;
                piece++;
            }
        }
        __syncwarp();
    } else {
        // ---------------- the eight finishing warps ----------------
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const int ctid = threadIdx.x;
        const Epilogue& ep = p.ep;
        const bool silu = (ep.steps & B200FC_STEP_SILU_MUL) != 0;
        bool ok = true;
        int piece = 0;
        long long it = it_begin;
        while (it < it_end) {
            const int rbk = (int)(it / p.spr);
            const int ks0 = (int)(it - (long long)rbk * p.spr);
            const int ks1 = (long long)(p.spr - ks0) < it_end - it ? p.spr : ks0 + (int)(it_end - it);
            const bool first_piece = it == it_begin;
            const int ab = piece & 1;
            it += ks1 - ks0;
            // post-op vectors of this row block (overlaps the wait for the accumulator)
            float ep_deq = 1.0f, ep_bias = 0.0f, ep_q = 1.0f;
            if (ctid < ROWS_PER_CTA) {
                const int n = p.n0 + rbk * ROWS_PER_CTA + ctid;
                if (n < p.n1) {
                    if (ep.steps & B200FC_STEP_DEQUANT) ep_deq = ep.deq_per_oc ? ep.deq_scale * ep.deq_per_oc[n] : ep.deq_scale;
                    if (ep.steps & B200FC_STEP_BIAS) ep_bias = ep.bias[n];
                    if (ep.steps & B200FC_STEP_QUANT) ep_q = ep.q_per_oc ? ep.q_per_oc[n] : ep.q_scale;
                }
            }
            consumer_sync();     // nobody still reads the previous piece's tile or vectors
            if (ctid < ROWS_PER_CTA) { s_ep[ctid] = ep_deq; s_ep[ROWS_PER_CTA + ctid] = ep_bias; s_ep[2 * ROWS_PER_CTA + ctid] = ep_q; }
            if (warp < 4) {
                ok = __all_sync(0xffffffffu, ok && mbar_wait(bar_acc_full + 8 * ab, (unsigned)(piece >> 1) & 1, abort_flag, limit));
                tc_fence_after();
                unsigned r[16];
                if (ok) {
                    tc_ld16(tmem_base + ((unsigned)(warp * 32) << 16) + (unsigned)(ab * 16), r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++) r[j] = 0u;
                }
                const int row = warp * 32 + lane;
#pragma unroll
                for (int j = 0; j < 16; j++) part[j * ROWS_PER_CTA + row] = __uint_as_float(r[j]);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty + 8 * ab);
            }
            piece++;
            consumer_sync();

            const bool whole = ks0 == 0 && ks1 == p.spr;
            bool finish = true;
            if (p.cluster) {
                finish = false;      // the pieces of the row block meet in distributed shared memory (end of the kernel)
            } else if (!whole) {
                const int nvec = p.M * ROWS_PER_CTA / 4;
                float4* slot = (float4*)(p.slots + (size_t)(2 * cta + (first_piece ? 0 : 1)) * SLOT_FLOATS);
                for (int v = ctid; v < nvec; v += CTHREADS) slot[v] = ((const float4*)part)[v];
                __threadfence();
                consumer_sync();
                const long long s_first = (long long)rbk * p.spr;
                const int c_first = piece_of(p, G, s_first), c_last = piece_of(p, G, s_first + p.spr - 1);
                if (ctid == 0) {
                    unsigned old;
                    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(p.counters + c_first) : "memory");
                    const bool last = old == (unsigned)(c_last - c_first);
                    if (last) p.counters[c_first] = 0;
                    *last_flag = last ? 1 : 0;
                }
                consumer_sync();
                finish = *last_flag != 0;
                if (finish) {
                    __threadfence();
                    const int which_first = piece_begin(p, G, c_first) < s_first ? 1 : 0;
                    const float4* base = (const float4*)p.slots;
                    for (int v = ctid; v < nvec; v += CTHREADS) {
                        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        for (int c = c_first; c <= c_last; c += 8) {
                            float4 t4[8];
#pragma unroll
                            for (int u = 0; u < 8; u++) {
                                const int cc = c + u;
                                const int which = cc == c_first ? which_first : 0;
                                t4[u] = cc <= c_last ? ld_gpu_f4(base + (size_t)(2 * cc + which) * (SLOT_FLOATS / 4) + v)
                                                     : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                            }
#pragma unroll
                            for (int u = 0; u < 8; u++) {
                                sum.x += t4[u].x; sum.y += t4[u].y; sum.z += t4[u].z; sum.w += t4[u].w;
                            }
                        }
                        ((float4*)part)[v] = sum;
                    }
                    consumer_sync();
                }
            }
            if (finish) {
                const int blk_row0 = p.n0 + rbk * ROWS_PER_CTA;
                const int out_rows = silu ? ROWS_PER_CTA / 2 : ROWS_PER_CTA;
                const int n_out = out_rows * p.M;
                for (int e = ctid; e < n_out; e += CTHREADS) {
                    const int tok = e / out_rows, orow = e % out_rows;
                    if (silu) {
                        const int grow = 32 * (orow >> 4) + (orow & 15);
                        if (blk_row0 + grow + 16 < p.n1) {
                            const float gsum = part[tok * ROWS_PER_CTA + grow], usum = part[tok * ROWS_PER_CTA + grow + 16];
                            unsigned short* crow = (unsigned short*)((char*)ep.C + (long long)tok * ep.ldc);
                            crow[(blk_row0 >> 1) + orow] = f32_to_bf16_bits(silu_f(gsum) * usum);
                        }
                    } else {
                        const int n = blk_row0 + orow;
                        if (n < p.n1) store_scalar(postop_staged(part[tok * ROWS_PER_CTA + orow], orow, ep.steps, s_ep), tok, n, ep);
                    }
                }
            }
        }
    }
    if (p.cluster) {
        // ---- aligned pieces launched as a cluster of S CTAs: every CTA finishes 1/S of the row block's outputs, adding the
        // partial tiles of all S CTAs in rank order (deterministic) ----
        __syncwarp();
        cluster_sync_all();
        const int S = p.S, rank = cta % S, blk_row0 = p.n0 + (cta / S) * ROWS_PER_CTA;
        const unsigned part_addr = smem_u32(part);
        const Epilogue& ep = p.ep;
        const bool silu = (ep.steps & B200FC_STEP_SILU_MUL) != 0;
        const int out_rows = silu ? ROWS_PER_CTA / 2 : ROWS_PER_CTA;
        const int n_out = out_rows * p.M;
        const int e_begin = (int)((long long)n_out * rank / S), e_end = (int)((long long)n_out * (rank + 1) / S);
        for (int e = e_begin + (int)threadIdx.x; e < e_end; e += TC_THREADS) {
            const int tok = e / out_rows, orow = e % out_rows;
            if (silu) {
                const int grow = 32 * (orow >> 4) + (orow & 15);
                float gsum = 0.0f, usum = 0.0f;
                for (int q = 0; q < S; q++) {
                    gsum += ld_peer_f32(part_addr + 4u * (unsigned)(tok * ROWS_PER_CTA + grow), (unsigned)q);
                    usum += ld_peer_f32(part_addr + 4u * (unsigned)(tok * ROWS_PER_CTA + grow + 16), (unsigned)q);
                }
                if (blk_row0 + grow + 16 < p.n1) {
                    unsigned short* crow = (unsigned short*)((char*)ep.C + (long long)tok * ep.ldc);
                    crow[(blk_row0 >> 1) + orow] = f32_to_bf16_bits(silu_f(gsum) * usum);
                }
            } else {
                float sum = 0.0f;
                for (int q = 0; q < S; q++) sum += ld_peer_f32(part_addr + 4u * (unsigned)(tok * ROWS_PER_CTA + orow), (unsigned)q);
                const int n = blk_row0 + orow;
                if (n < p.n1) store_scalar(postop_staged(sum, orow, ep.steps, s_ep), tok, n, ep);
            }
        }
        cluster_sync_all();  // nobody leaves while a peer may still read its partial tile
    }
    tc_fence_before();
    __syncthreads();
    if (warp == CWARPS + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32u) : "memory");
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, 3);
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

int device_sms() {
    int dev = 0, n = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n > 0 ? n : 148;
}

template <int WB, int NT>
int launch_variant(const CUtensorMap& map, const Params& p_in, int grid, cudaStream_t s) {
    const int cluster = p_in.cluster ? p_in.S : 1;
    using L = Layout<WB, NT>;
    static_assert(L::MP * L::XROW >= 2 * ROWS_PER_CTA * L::MP * 4, "partial tiles must fit the activation buffer");
    static std::atomic<unsigned long long> attr_devices{0};
    {
        const int arc = once_per_device(attr_devices, [] {
            B200FC_CUDA(cudaFuncSetAttribute(gemv_tma_kernel<WB, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM));
            return (int)B200FC_OK;
        });
        if (arc) return arc;
    }
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    Params p = p_in;
    p.ximg = nullptr;
    if constexpr (WB != 16) {
        // Pre-converted activations pay from about two chunks per CTA on (they add a small launch to the chain).
        static int force_img = -1;
        if (force_img < 0) { const char* e = getenv("B200FC_GEMV_XIMG"); force_img = e ? (atoi(e) ? 1 : 0) : 2; }
        constexpr int SPC = L::CHUNK / (STAGE_K_BYTES * 8 / WB);
        const bool use_img = force_img == 2 ? (p.total / grid >= 2 * SPC) : force_img == 1;
        if (use_img) {
            const int n_chunks = (p.spr + SPC - 1) / SPC;
            void* img = nullptr;
            int rc = get_stream_scratch((size_t)n_chunks * L::MP * L::XROW, s, 6, &img);
            if (rc) return rc;
            cudaLaunchConfig_t c0 = {};
            c0.gridDim = dim3(n_chunks, 1, 1);
            c0.blockDim = dim3(CTHREADS, 1, 1);
            c0.stream = s;
            c0.attrs = attr;
            c0.numAttrs = 1;
            B200FC_CUDA(cudaLaunchKernelEx(&c0, xstage_kernel<WB, NT>, p.X, p.ldx, p.M, p.K, (unsigned char*)img));
            count_launch();
            p.ximg = (const unsigned char*)img;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = L::SMEM;
    cfg.stream = s;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    B200FC_CUDA(cudaLaunchKernelEx(&cfg, gemv_tma_kernel<WB, NT>, map, p));
    count_launch();
    return B200FC_OK;
}

}  // namespace

#ifdef B200FC_TRACE
static unsigned long long* g_trace_ptr = nullptr;
extern "C" void* b200fc_debug_trace_ptr(void) { return g_trace_ptr; }
#endif

size_t gemv_scratch_bytes() { return (size_t)kGemvMaxCtas * (2 * SLOT_FLOATS * sizeof(float) + sizeof(unsigned)); }

// validation, tensor map and the parameters that do not depend on how the work is cut
static int prepare_job(const Weight& w, const void* A, int M, int K, int64_t lda, int n0, int n1, const Epilogue& ep,
                       cudaStream_t s, void*& scratch, CUtensorMap& map, Params& p, int& row_blocks) {
    if (M < 1 || M > 16) { set_error("gemv: M must be in [1, 16]"); return B200FC_ERR_INVALID; }
    if (w.dtype == B200FC_U8) { set_error("gemv: unsigned 8-bit weights are not supported with bf16 activations"); return B200FC_ERR_UNSUPPORTED; }
    if ((ep.steps & B200FC_STEP_SILU_MUL) && (n0 % 32)) { set_error("gemv: SILU_MUL needs n0 %% 32 == 0"); return B200FC_ERR_INVALID; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled entry point not available"); return B200FC_ERR_CUDA; }
    // the packed weights as a byte matrix [N_pad, K_pad bytes]; box = 128 bytes of K x 128 rows, 128-byte swizzle
    cuuint64_t dims[2] = {(cuuint64_t)w.ld_bytes(), (cuuint64_t)w.N_pad};
    cuuint64_t strides[1] = {(cuuint64_t)w.ld_bytes()};
    cuuint32_t box[2] = {STAGE_K_BYTES, ROWS_PER_CTA};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w.data, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d)", (int)r); return B200FC_ERR_CUDA; }

    p.spr = (int)(w.ld_bytes() / STAGE_K_BYTES);
    row_blocks = (n1 - n0 + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
    p.total = (long long)row_blocks * p.spr;
    p.X = (const unsigned char*)A;
    p.ldx = lda;
    p.M = M; p.K = K;
    p.n0 = n0; p.n1 = n1;
    p.ep = ep;
    p.status = kernel_status_word();
    if (!p.status) { set_error("gemv: no kernel status word on this device"); return B200FC_ERR_CUDA; }
    p.wait_limit_ns = wait_limit_ns();
    p.S = 0; p.cluster = 0; p.pf_cap = 0;
    p.ximg = nullptr;
#ifdef B200FC_TRACE
    {
        static unsigned long long* tr = nullptr;
        static int launches = 0;
        if (!tr) {
            if (cudaMalloc(&tr, 64 * 320 * 8 * 8) != cudaSuccess) { set_error("trace buffer"); return B200FC_ERR_NOMEM; }
            cudaMemset(tr, 0, 64 * 320 * 8 * 8);
        }
        p.trace = tr; p.trace_launch = launches++;
        g_trace_ptr = tr;
    }
#endif
    if (!scratch) {
        int rc = get_gemv_scratch(s, &scratch);
        if (rc) return rc;
    }
    p.counters = (unsigned*)scratch;
    p.slots = (float*)((char*)scratch + (size_t)kGemvMaxCtas * sizeof(unsigned));
    p.scales = w.scale_grp;
    return B200FC_OK;
}

// environment switches, for experiments
static int g_pf_cap = -1, g_per_sm = 2, g_force_stream = 0, g_force_aligned = 0;
static void read_switches() {
    if (g_pf_cap >= 0) return;
    const char* e = getenv("B200FC_GEMV_CTAS_PER_SM");   // 1 leaves the second resident place to the next kernel
    g_per_sm = (e && atoi(e) == 1) ? 1 : 2;
    e = getenv("B200FC_GEMV_STREAMK");                   // 1: never align pieces with row blocks
    g_force_stream = (e && atoi(e) == 1) ? 1 : 0;
    g_force_aligned = (e && atoi(e) == 2) ? 1 : 0;       // 2: align whenever the row blocks fit the grid
    e = getenv("B200FC_GEMV_PREFETCH");                  // stages prefetched into L2 at CTA start (0 = none)
    int v = e ? atoi(e) : 0;
    g_pf_cap = v < 0 ? 0 : (v > 64 ? 64 : v);
}

static std::atomic<int> g_per_sm_api{0};      // b200fc_set_decode_ctas_per_sm: 0 = the default / the environment's choice
void set_decode_ctas_per_sm(int n) { g_per_sm_api.store(n); }

static long long max_ctas() {
    int sms = device_sms();
    if (sm_limit() > 0 && sm_limit() < sms) sms = sm_limit();
    const int api = g_per_sm_api.load();
    long long gmax = (long long)sms * (api == 1 || api == 2 ? api : g_per_sm);
    return gmax > kGemvMaxCtas - 2 ? kGemvMaxCtas - 2 : gmax;   // the last two counter words serve the two-job barrier
}

static int launch_tc(const CUtensorMap& map_w, const Params& p, const void* A, int M, int K, int64_t lda, int grid, cudaStream_t s) {
    EncodeTiledFn fn = encode_fn();
    // the activations as a bf16 matrix [M, K]; box = 64 K x 16 tokens, rows past M and columns past K read as zeros
    CUtensorMap map_x;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    cuuint64_t strides[1] = {(cuuint64_t)lda};
    cuuint32_t box[2] = {STAGE_K_BYTES / 2, 16};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)A, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (activations) failed (%d)", (int)r); return B200FC_ERR_CUDA; }
    static std::atomic<unsigned long long> attr_devices{0};
    {
        const int arc = once_per_device(attr_devices, [] {
            B200FC_CUDA(cudaFuncSetAttribute(gemv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TcLayout::SMEM));
            return (int)B200FC_OK;
        });
        if (arc) return arc;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(TC_THREADS, 1, 1);
    cfg.dynamicSmemBytes = TcLayout::SMEM;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = p.cluster ? p.S : 1;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    B200FC_CUDA(cudaLaunchKernelEx(&cfg, gemv_tc_kernel, map_w, map_x, p));
    count_launch();
    return B200FC_OK;
}

int launch_gemv_tma(const Weight& w, const void* A, int M, int K, int64_t lda, int n0, int n1, const Epilogue& ep,
                    cudaStream_t s, void* scratch) {
    if (n1 <= n0 && M >= 1 && M <= 16) return B200FC_OK;
    CUtensorMap map;
    Params p;
    int row_blocks = 0;
    int rc = prepare_job(w, A, M, K, lda, n0, n1, ep, s, scratch, map, p, row_blocks);
    if (rc) return rc;
    read_switches();
    p.pf_cap = g_pf_cap;
    const long long gmax = max_ctas();
    // Three ways to cut the work; the cost model counts the stages of the longest CTA plus the time of the reduction
    // that follows, in units of one stage's streaming time.
    //   stream-K: equal pieces whatever the shape; a CTA may hold the end of one row block and the start of the next,
    //             partial sums meet through the global scratch (several round trips to L2, twice for such a CTA);
    //   aligned:  S pieces per row block, one per CTA.  S = 1 needs no reduction; 2 <= S <= 8 runs as clusters of S CTAs
    //             whose partial sums meet in distributed shared memory (fast, so this wins for small matrices).
    long long grid = gmax < p.total / 2 ? gmax : p.total / 2;
    if (grid < 1) grid = 1;
    long long best = (p.total + grid - 1) / grid + 6;
    if (!g_force_stream && row_blocks <= gmax) {
        int S = (int)(gmax / row_blocks);
        if (S > 8) S = 8;
        if (S > p.spr / 2) S = p.spr / 2;
        if (S < 1) S = 1;
        const long long cost = (p.spr + S - 1) / S + (S > 1 ? 1 : 0);
        if (cost <= best || g_force_aligned) { best = cost; p.S = S; p.cluster = S > 1 ? 1 : 0; grid = (long long)row_blocks * S; }
    }
    if (w.dtype == B200FC_S4) {
        if (!w.scale_grp || (n0 % ROWS_PER_CTA)) { set_error("gemv: 4-bit weights need group scales and n0 %% 128 == 0"); return B200FC_ERR_INVALID; }
        return M <= 8 ? launch_variant<4, 1>(map, p, (int)grid, s) : launch_variant<4, 2>(map, p, (int)grid, s);
    }
    if (w.dtype == B200FC_BF16 && (((uintptr_t)A | (uintptr_t)lda) & 15) == 0) {
        // Measured (Llama-7B MLP, decode): 58.6 against 61.6 us at M = 16, 53.3 against 51.2 us at M = 1 — the tensor-memory
        // path costs a token column nothing but pays a little for its activation tiles at every stage, so it takes the
        // calls with more than 8 rows.  B200FC_GEMV_TC=0 never uses it, =2 always.
        static int use_tc = -1;
        if (use_tc < 0) { const char* e = getenv("B200FC_GEMV_TC"); use_tc = e ? atoi(e) : 1; }
        if (use_tc == 2 || (use_tc == 1 && M > 8)) return launch_tc(map, p, A, M, K, lda, (int)grid, s);
    }
    const bool w8 = w.dtype == B200FC_S8;
    if (M <= 8) return w8 ? launch_variant<8, 1>(map, p, (int)grid, s) : launch_variant<16, 1>(map, p, (int)grid, s);
    return w8 ? launch_variant<8, 2>(map, p, (int)grid, s) : launch_variant<16, 2>(map, p, (int)grid, s);
}

template <int NT>
static int launch_mlp_variant(const CUtensorMap& m1, const CUtensorMap& m2, const Params& p1, const Params& p2, int grid,
                              cudaStream_t s) {
    using L = Layout<16, NT>;
    static std::atomic<unsigned long long> attr_devices{0};
    static std::atomic<int> resident{0};     // CTAs of this kernel an SM holds (all CTAs of the grid must be resident)
    {
        const int arc = once_per_device(attr_devices, [] {
            B200FC_CUDA(cudaFuncSetAttribute(mlp_decode_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM));
            int n = 0;
            B200FC_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, mlp_decode_kernel<NT>, THREADS, L::SMEM));
            resident.store(n);
            return (int)B200FC_OK;
        });
        if (arc) return arc;
    }
    if ((long long)resident.load() * device_sms() < grid) return B200FC_ERR_UNSUPPORTED;   // caller falls back to two launches
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = L::SMEM;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200FC_CUDA(cudaLaunchKernelEx(&cfg, mlp_decode_kernel<NT>, m1, m2, p1, p2));
    count_launch();
    return B200FC_OK;
}

// Decode-shaped MLP (bf16 weights, M <= 16) as ONE launch: job 1 = gate/up with the SiLU*up store into `act`
// ([M, ns] bf16), job 2 = down over `act`.  Both jobs are cut stream-K over the same grid (no clusters: the CTAs of a
// job meet through the global scratch), and the CTAs wait for one another between the jobs, so the whole grid must be
// resident: at most two CTAs per SM, and the SM limit of the GEMMs is not honoured.  Returns B200FC_ERR_UNSUPPORTED
// (without an error message) when the shape or the device does not allow it; the caller then launches twice.
int launch_mlp_decode_fused(const Weight& gate_up, const Weight& down, const void* x, int64_t ldx, int M, int K, int ns,
                            void* act, const Epilogue& ep_down, cudaStream_t s, void* scratch) {
    if (gate_up.dtype != B200FC_BF16 || down.dtype != B200FC_BF16 || M < 1 || M > 16) return B200FC_ERR_UNSUPPORTED;
    if (sm_limit() > 0 && sm_limit() < device_sms()) return B200FC_ERR_UNSUPPORTED;
    static int enabled = -1;
    // Off unless B200FC_MLP_FUSED=1: measured slower than two launches (Llama-7B MLP, M = 1: 57.6 vs 51.5 us) — the second
    // job cannot use the cluster reduction (a grid of clusters would not be resident as a whole), which alone costs 3.5 us,
    // and the barrier between the jobs with its fences costs more than the programmatic launch edge it replaces.
    if (enabled < 0) { const char* e = getenv("B200FC_MLP_FUSED"); enabled = (e && atoi(e)) ? 1 : 0; }
    if (!enabled) return B200FC_ERR_UNSUPPORTED;
    Epilogue ep1 = {};
    ep1.steps = B200FC_STEP_SILU_MUL; ep1.out_dtype = B200FC_BF16; ep1.C = act; ep1.ldc = (long long)ns * 2;
    ep1.deq_scale = 1.0f; ep1.q_scale = 1.0f;
    CUtensorMap m1, m2;
    Params p1, p2;
    int rb1 = 0, rb2 = 0;
    int rc = prepare_job(gate_up, x, M, K, ldx, 0, 2 * ns, ep1, s, scratch, m1, p1, rb1);
    if (rc) return rc;
    rc = prepare_job(down, act, M, ns, (int64_t)ns * 2, 0, K, ep_down, s, scratch, m2, p2, rb2);
    if (rc) return rc;
    read_switches();
    long long grid = (long long)device_sms() * 2;
    if (grid > kGemvMaxCtas - 2) grid = kGemvMaxCtas - 2;
    // every CTA needs at least two stages of either job for the piece arithmetic (and the launch is pointless below that)
    if (p1.total < 2 * grid || p2.total < 2 * grid) return B200FC_ERR_UNSUPPORTED;
    return M <= 8 ? launch_mlp_variant<1>(m1, m2, p1, p2, (int)grid, s) : launch_mlp_variant<2>(m1, m2, p1, p2, (int)grid, s);
}

}  // namespace b200fc
