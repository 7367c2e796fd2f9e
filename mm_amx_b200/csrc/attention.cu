// Decode attention: one query token per sequence and head against a bf16 key/value cache — an HBM-bound stream of K and V.
//
// Grown from the reference's two pieces: the w = query x Key^T mat-vec on the AMX unit (MatMulVec_AMX, test_jit.cpp:17-95;
// MatmulVector, include/kernels_amx.hpp:959-1042) and its one-token attention that cuts the key range into blocks,
// encodes each block into a sub-state (score maximum, sum of exponentials, weighted values) and combines the
// sub-states afterwards (MHA2Kernels, include/kernels_mha.hpp:146-270; fp32 AVX2, softmax without a scale factor).
//
// How the bytes move
//   grid = (splits, kv heads, sequences); a CTA owns one contiguous token range of one (sequence, kv head) and all G = H / Hkv
//   query heads that share it, so K and V cross HBM once however many query heads read them.  The four warps of a CTA work
//   independently on alternating 16-token blocks: each keeps a ring of STAGES blocks (K and V rows, 16-byte cp.async,
//   XOR-swizzled so that ldmatrix is conflict-free) in flight and never waits for another warp inside the loop.
//   Per block: S^T[16 heads x 16 tokens] = Q K^T with mma.sync.m16n8k16 (Q fragments stay in registers, K fragments by
//   ldmatrix), online softmax per head in the exp2 domain, P rounded to bf16 straight from the accumulator registers
//   into the A operand of O[16 heads x D] += P V (V fragments by ldmatrix.trans).
//   At the end the four warps' states meet in shared memory; with one split the CTA normalises and stores, otherwise it
//   writes its sub-state (maximum, sum, unnormalised values) to a workspace and a second small kernel, launched as a
//   programmatic dependent, combines the splits — the reference's "combine sub-states" step.
#include <cuda_bf16.h>
#include <cstdlib>
#include "common.cuh"

namespace b200fc {

namespace {

constexpr int ATT_WARPS = 4;
constexpr int ATT_THREADS = ATT_WARPS * 32;
constexpr int BLK = 16;            // tokens per block (one k-step of the P V product)
constexpr int ATT_STAGES = 3;
constexpr int MAX_SPLITS = 64;

struct AttnParams {
    const unsigned char* q; long long q_bs, q_hs;          // bytes
    const unsigned char* k; const unsigned char* v;
    long long kv_bs, kv_hs, kv_ts;                          // bytes
    void* out; long long o_bs, o_hs; int out_f32;
    const int* seq_lens;                                    // optional [B]
    int H, Hkv, G, N;
    int tokens_per_split, splits;
    float scale_log2e;                                      // scale * log2(e)
    float* ws_o;                                            // [B][H][splits][D]
    float* ws_ml;                                           // [B][H][splits][2]
};

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(unsigned dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                               unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *(unsigned*)&h;
}

// shared memory of one CTA: per warp a ring of STAGES x (K block, V block); reused for the warps' states at the end
template <int D> struct AttnSmem {
    static constexpr int ROW = D * 2;                       // bytes per token row
    static constexpr int BLOCK_BYTES = BLK * ROW;           // K (or V) rows of one block
    static constexpr int STAGE_BYTES = 2 * BLOCK_BYTES;
    static constexpr int WARP_BYTES = ATT_STAGES * STAGE_BYTES;
    static constexpr int RING = ATT_WARPS * WARP_BYTES;
    static constexpr int STATE = ATT_WARPS * 16 * D * 4 + ATT_WARPS * 16 * 2 * 4;
    static constexpr int BYTES = (RING > STATE ? RING : STATE) + 128;
};

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 2) decode_attention_kernel(const AttnParams p) {
    using SM = AttnSmem<D>;
    constexpr int CHUNKS = D / 8;          // 16-byte chunks per token row
    constexpr int KSTEPS = D / 16;
    extern __shared__ unsigned char att_smem_raw[];
    // aligned by pointer arithmetic on the __shared__ array (an integer round trip would turn every access generic)
    unsigned char* smem = att_smem_raw + (((smem_addr(att_smem_raw) + 127u) & ~127u) - smem_addr(att_smem_raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
    const int G = p.G;

    // the next kernel of the stream (the combine step, or whatever follows) may start its prologue
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // q, the cache and the workspace may be written by the previous kernel of the stream
    asm volatile("griddepcontrol.wait;" ::: "memory");

    int len = p.N;
    if (p.seq_lens) { len = p.seq_lens[b]; len = len < 0 ? 0 : (len > p.N ? p.N : len); }
    const int n_begin = split * p.tokens_per_split;
    int n_end = n_begin + p.tokens_per_split;
    n_end = n_end > len ? len : n_end;
    const int nblocks = n_end > n_begin ? (n_end - n_begin + BLK - 1) / BLK : 0;

    const unsigned char* kbase = p.k + (long long)b * p.kv_bs + (long long)hkv * p.kv_hs;
    const unsigned char* vbase = p.v + (long long)b * p.kv_bs + (long long)hkv * p.kv_hs;
    unsigned char* ring = smem + warp * SM::WARP_BYTES;

    // issue the loads of this warp's block j (block index inside the CTA's range: warp + j * ATT_WARPS)
    auto issue = [&](int j) {
        const int blk = warp + j * ATT_WARPS;
        if (blk < nblocks) {
            const int tok0 = n_begin + blk * BLK;
            unsigned char* st = ring + (j % ATT_STAGES) * SM::STAGE_BYTES;
            // BLK rows x CHUNKS chunks for K and the same for V; rows past the end repeat the last valid token
#pragma unroll
            for (int i = 0; i < BLK * CHUNKS / 32; i++) {
                const int u = i * 32 + lane, row = u / CHUNKS, c = u % CHUNKS;
                int tok = tok0 + row;
                tok = tok < n_end ? tok : n_end - 1;
                const unsigned dst = smem_addr(st + row * SM::ROW + ((c ^ (row & 7)) << 4));
                cp_async16(dst, kbase + (long long)tok * p.kv_ts + c * 16);
                cp_async16(dst + SM::BLOCK_BYTES, vbase + (long long)tok * p.kv_ts + c * 16);
            }
        }
        cp_async_commit();   // always, so that the group count stays in step
    };

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};   // rows g and g + 8 (the lane's partial sums of l)

    const int my_blocks = nblocks > warp ? (nblocks - warp + ATT_WARPS - 1) / ATT_WARPS : 0;
#pragma unroll
    for (int j = 0; j < ATT_STAGES - 1; j++) issue(j);

    // (the first blocks of K and V are on their way: the latency of the query loads hides under theirs)
    // ---- Q fragments: rows = the G query heads of this kv head (padded to 16 with zeros) ----
    unsigned qa[KSTEPS][4];
    {
        const unsigned char* qb = p.q + (long long)b * p.q_bs + (long long)(hkv * G) * p.q_hs;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            const int d0 = ks * 16 + 2 * t;
            qa[ks][0] = g < G ? *(const unsigned*)(qb + (long long)g * p.q_hs + d0 * 2) : 0u;
            qa[ks][1] = g + 8 < G ? *(const unsigned*)(qb + (long long)(g + 8) * p.q_hs + d0 * 2) : 0u;
            qa[ks][2] = g < G ? *(const unsigned*)(qb + (long long)g * p.q_hs + (d0 + 8) * 2) : 0u;
            qa[ks][3] = g + 8 < G ? *(const unsigned*)(qb + (long long)(g + 8) * p.q_hs + (d0 + 8) * 2) : 0u;
        }
    }


    for (int j = 0; j < my_blocks; j++) {
        issue(j + ATT_STAGES - 1);
        cp_async_wait<ATT_STAGES - 1>();
        __syncwarp();
        const unsigned char* st = ring + (j % ATT_STAGES) * SM::STAGE_BYTES;
        const unsigned kst = smem_addr(st), vst = kst + SM::BLOCK_BYTES;
        const int tok0 = n_begin + (warp + j * ATT_WARPS) * BLK;

        // ---- S^T = Q K^T: [16 heads x 16 tokens] as two 8-token tiles ----
        float s[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
        {
            const int mi = lane >> 3, r = lane & 7;
            const int tok = (mi >> 1) * 8 + r;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks++) {
                unsigned kb[4];
                ldsm_x4(kb, kst + tok * SM::ROW + (((2 * ks + (mi & 1)) ^ (tok & 7)) << 4));
                mma_bf16_16816(s[0], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], kb[0], kb[1]);
                mma_bf16_16816(s[1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], kb[2], kb[3]);
            }
        }
        // ---- online softmax (exp2 domain); tokens past the end count as -inf ----
        float bm[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int tt = 0; tt < 2; tt++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int tok = tok0 + tt * 8 + 2 * t + (c & 1);
                const float v = tok < n_end ? s[tt][c] * p.scale_log2e : -INFINITY;
                s[tt][c] = v;
                bm[c >> 1] = fmaxf(bm[c >> 1], v);
            }
#pragma unroll
        for (int r = 0; r < 2; r++) {
            bm[r] = fmaxf(bm[r], __shfl_xor_sync(0xffffffffu, bm[r], 1));
            bm[r] = fmaxf(bm[r], __shfl_xor_sync(0xffffffffu, bm[r], 2));
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const float m_new = fmaxf(m_run[r], bm[r]);          // finite: every block has at least one valid token
            corr[r] = exp2f(m_run[r] - m_new);                   // 0 on the first block (m_run = -inf)
            m_run[r] = m_new;
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int tt = 0; tt < 2; tt++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const float e = exp2f(s[tt][c] - m_run[c >> 1]);
                s[tt][c] = e;
                l_run[c >> 1] += e;
            }
        const unsigned pa0 = pack_bf16x2(s[0][0], s[0][1]), pa1 = pack_bf16x2(s[0][2], s[0][3]);
        const unsigned pa2 = pack_bf16x2(s[1][0], s[1][1]), pa3 = pack_bf16x2(s[1][2], s[1][3]);
        // ---- O = O * corr + P V ----
        {
            const int mi = lane >> 3, r = lane & 7;
            const int tok = (mi & 1) * 8 + r;
#pragma unroll
            for (int c2 = 0; c2 < CHUNKS / 2; c2++) {
                unsigned vb[4];
                ldsm_x4_trans(vb, vst + tok * SM::ROW + (((2 * c2 + (mi >> 1)) ^ (tok & 7)) << 4));
#pragma unroll
                for (int h2 = 0; h2 < 2; h2++) {
                    float (&acc)[4] = o[2 * c2 + h2];
                    acc[0] *= corr[0]; acc[1] *= corr[0]; acc[2] *= corr[1]; acc[3] *= corr[1];
                    mma_bf16_16816(acc, pa0, pa1, pa2, pa3, vb[2 * h2], vb[2 * h2 + 1]);
                }
            }
        }
        __syncwarp();   // every lane is done with the stage before the next issue overwrites it
    }
    cp_async_wait<0>();

    // the lane's partial sums of l cover its own token columns: add the four lanes of a row
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }

    // ---- the four warps' states meet in shared memory (over the rings) ----
    __syncthreads();
    float* st_o = (float*)smem;                                   // [warp][16 heads][D]
    float* st_ml = st_o + ATT_WARPS * 16 * D;                     // [warp][16 heads][2]
#pragma unroll
    for (int i = 0; i < D / 8; i++) {
        float* base = st_o + (warp * 16) * D + i * 8 + 2 * t;
        *(float2*)(base + g * D) = make_float2(o[i][0], o[i][1]);
        *(float2*)(base + (g + 8) * D) = make_float2(o[i][2], o[i][3]);
    }
    if (t == 0) {
        st_ml[(warp * 16 + g) * 2] = m_run[0]; st_ml[(warp * 16 + g) * 2 + 1] = l_run[0];
        st_ml[(warp * 16 + g + 8) * 2] = m_run[1]; st_ml[(warp * 16 + g + 8) * 2 + 1] = l_run[1];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < G * D; e += ATT_THREADS) {
        const int h = e / D, d = e % D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) m = fmaxf(m, st_ml[(w * 16 + h) * 2]);
        float l = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) {
            const float mw = st_ml[(w * 16 + h) * 2];
            const float f = mw == -INFINITY ? 0.0f : exp2f(mw - m);
            l = fmaf(st_ml[(w * 16 + h) * 2 + 1], f, l);
            acc = fmaf(st_o[(w * 16 + h) * D + d], f, acc);
        }
        const int head = hkv * G + h;
        if (p.splits == 1) {
            const float r = l > 0.0f ? acc / l : 0.0f;            // an empty sequence yields zeros
            char* orow = (char*)p.out + (long long)b * p.o_bs + (long long)head * p.o_hs;
            if (p.out_f32) ((float*)orow)[d] = r;
            else ((unsigned short*)orow)[d] = f32_to_bf16_bits(r);
        } else {
            const size_t idx = ((size_t)b * p.H + head) * p.splits + split;
            p.ws_o[idx * D + d] = acc;
            if (d == 0) { p.ws_ml[idx * 2] = m; p.ws_ml[idx * 2 + 1] = l; }
        }
    }
}

// combines the sub-states of the splits: grid (H, B), D threads
template <int D>
__global__ void __launch_bounds__(D) attention_combine_kernel(const AttnParams p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    const size_t base = ((size_t)b * p.H + head) * p.splits;
    float m = -INFINITY;
    for (int sp = 0; sp < p.splits; sp++) m = fmaxf(m, p.ws_ml[(base + sp) * 2]);
    float l = 0.0f, acc = 0.0f;
    for (int sp = 0; sp < p.splits; sp++) {
        const float ms = p.ws_ml[(base + sp) * 2];
        const float f = ms == -INFINITY ? 0.0f : exp2f(ms - m);
        l = fmaf(p.ws_ml[(base + sp) * 2 + 1], f, l);
        acc = fmaf(p.ws_o[(base + sp) * D + d], f, acc);
    }
    const float r = l > 0.0f ? acc / l : 0.0f;
    char* orow = (char*)p.out + (long long)b * p.o_bs + (long long)head * p.o_hs;
    if (p.out_f32) ((float*)orow)[d] = r;
    else ((unsigned short*)orow)[d] = f32_to_bf16_bits(r);
}

template <int D>
int launch_attention_d(AttnParams& p, int B, cudaStream_t s) {
    using SM = AttnSmem<D>;
    static std::atomic<unsigned long long> attr_devices{0};
    {
        const int arc = once_per_device(attr_devices, [] {
            B200FC_CUDA(cudaFuncSetAttribute(decode_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::BYTES));
            return (int)B200FC_OK;
        });
        if (arc) return arc;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.splits, p.Hkv, B);
    cfg.blockDim = dim3(ATT_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SM::BYTES;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200FC_CUDA(cudaLaunchKernelEx(&cfg, decode_attention_kernel<D>, (const AttnParams)p));
    count_launch();
    if (p.splits > 1) {
        cfg.gridDim = dim3(p.H, B, 1);
        cfg.blockDim = dim3(D, 1, 1);
        cfg.dynamicSmemBytes = 0;
        B200FC_CUDA(cudaLaunchKernelEx(&cfg, attention_combine_kernel<D>, (const AttnParams)p));
        count_launch();
    }
    return B200FC_OK;
}

}  // namespace

int launch_decode_attention(const b200fc_attention_t& a, cudaStream_t s) {
    if (!a.q || !a.k || !a.v || !a.out) { set_error("decode_attention: null pointer"); return B200FC_ERR_INVALID; }
    if (a.B < 0 || a.H <= 0 || a.Hkv <= 0 || a.N < 0 || (a.H % a.Hkv) || a.H / a.Hkv > 16) {
        set_error("decode_attention: need H %% Hkv == 0 and at most 16 query heads per kv head");
        return B200FC_ERR_INVALID;
    }
    if (a.B > 65535 || a.Hkv > 65535) { set_error("decode_attention: at most 65535 sequences and kv heads per call"); return B200FC_ERR_INVALID; }
    if (a.D != 64 && a.D != 128) { set_error("decode_attention: head size must be 64 or 128"); return B200FC_ERR_UNSUPPORTED; }
    if (a.out_dtype != B200FC_BF16 && a.out_dtype != B200FC_F32) { set_error("decode_attention: out_dtype must be bf16 or f32"); return B200FC_ERR_INVALID; }
    if (((uintptr_t)a.k & 15) || ((uintptr_t)a.v & 15) || (a.kv_batch_stride & 15) || (a.kv_head_stride & 15) || (a.kv_token_stride & 15) ||
        a.kv_token_stride < (int64_t)a.D * 2) {
        set_error("decode_attention: the cache needs 16-byte aligned pointers and strides, token stride >= D * 2");
        return B200FC_ERR_INVALID;
    }
    if (((uintptr_t)a.q & 3) || (a.q_batch_stride & 3) || (a.q_head_stride & 3) || ((uintptr_t)a.out & 3) || (a.out_batch_stride & 3) || (a.out_head_stride & 3)) {
        set_error("decode_attention: q and out need 4-byte aligned pointers and strides");
        return B200FC_ERR_INVALID;
    }
    if (a.B == 0) return B200FC_OK;
    AttnParams p;
    p.q = (const unsigned char*)a.q; p.q_bs = a.q_batch_stride; p.q_hs = a.q_head_stride;
    p.k = (const unsigned char*)a.k; p.v = (const unsigned char*)a.v;
    p.kv_bs = a.kv_batch_stride; p.kv_hs = a.kv_head_stride; p.kv_ts = a.kv_token_stride;
    p.out = a.out; p.o_bs = a.out_batch_stride; p.o_hs = a.out_head_stride; p.out_f32 = a.out_dtype == B200FC_F32;
    p.seq_lens = a.seq_lens;
    p.H = a.H; p.Hkv = a.Hkv; p.G = a.H / a.Hkv; p.N = a.N;
    p.scale_log2e = a.scale * 1.4426950408889634f;
    // splits: as many as still give ONE round of two CTAs per SM (measured: a ragged second round costs more than a
    // partly filled first one; 96 KB in flight per CTA saturate HBM from ~130 CTAs on), at least two 16-token blocks per
    // warp and split
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    static int force_splits = -1;
    if (force_splits < 0) { const char* e = getenv("B200FC_ATTN_SPLITS"); force_splits = e ? atoi(e) : 0; }
    const long long pairs = (long long)a.B * a.Hkv;
    int splits = (int)(2LL * sms / pairs);
    const int max_by_len = (a.N + 2 * BLK * ATT_WARPS - 1) / (2 * BLK * ATT_WARPS);
    if (splits > max_by_len) splits = max_by_len;
    if (force_splits > 0) splits = force_splits;
    if (splits > MAX_SPLITS) splits = MAX_SPLITS;
    if (splits < 1) splits = 1;
    int tps = (a.N + splits - 1) / splits;
    tps = (tps + BLK - 1) / BLK * BLK;
    if (tps < BLK) tps = BLK;
    splits = a.N > 0 ? (a.N + tps - 1) / tps : 1;
    p.tokens_per_split = tps; p.splits = splits;
    p.ws_o = nullptr; p.ws_ml = nullptr;
    if (splits > 1) {
        const size_t n_sub = (size_t)a.B * a.H * splits;
        void* ws = nullptr;
        int rc = get_stream_scratch(n_sub * (a.D + 2) * sizeof(float), s, 5, &ws);
        if (rc) return rc;
        p.ws_o = (float*)ws;
        p.ws_ml = p.ws_o + n_sub * a.D;
    }
    return a.D == 128 ? launch_attention_d<128>(p, a.B, s) : launch_attention_d<64>(p, a.B, s);
}

}  // namespace b200fc
