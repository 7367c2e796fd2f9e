/*
 * b200fc — C ABI of the B200 (sm_100a) fully-connected / Llama-MLP engine that stands in for the CPU kernels of
 * usstq/mm_amx.  Every entry point below replaces one interface of the reference; the citation gives the
 * reference file:line (paths relative to the mm_amx tree).
 *
 * Conventions
 *   - plain pointers and sizes only; all strides are in BYTES (tensor2D::stride, include/tensor2D.hpp:34);
 *   - matrices are row-major; bf16 is the upper half of an IEEE fp32 (ov::bfloat16, include/bf16.hpp:18);
 *   - unless a function name ends in _host, data pointers are DEVICE pointers of the current CUDA device and the
 *     call is asynchronous on `stream` (a cudaStream_t passed as void*, NULL = default stream);
 *   - every function returns a b200fc_status_t; b200fc_last_error() gives the message of the calling thread's last
 *     failure.  Nothing aborts the process (the reference asserts / aborts, include/misc.hpp:289-293).
 *   - there is no CPU fallback: without a CUDA device every compute call fails with B200FC_ERR_CUDA.
 */
#ifndef B200FC_H
#define B200FC_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    B200FC_OK = 0,
    B200FC_ERR_INVALID = 1,     /* bad argument (shape, stride, alignment, dtype combination) */
    B200FC_ERR_CUDA = 2,        /* a CUDA runtime / driver call failed */
    B200FC_ERR_UNSUPPORTED = 3, /* valid in the reference, not implemented here */
    B200FC_ERR_NOMEM = 4,
    B200FC_ERR_KERNEL = 5       /* a kernel reported a bounded wait that ran out */
} b200fc_status_t;

typedef enum {
    B200FC_BF16 = 0, B200FC_S8 = 1, B200FC_U8 = 2, B200FC_F32 = 3, B200FC_S32 = 4,
    B200FC_S4 = 5   /* only as the stored type of B200FC_PACK_INT4_GROUP weights (two values per byte) */
} b200fc_dtype_t;

/* Post-op steps, executed in this fixed order (amx_kernel::PP::Steps, include/kernels_amx.hpp:540-550, and
 * PP::BiasGeluStore::operator(), :586-672):  [int32 accumulator -> fp32] -> DEQUANT -> BIAS -> GELU -> QUANT -> store.
 * SILU_MUL is this library's addition for the fused MLP (runGateUp, tests/amx-mlp.cpp:707-737): the weight rows
 * come in groups of 32 = 16 gate rows followed by the 16 up rows of the same channels, and the store writes
 * silu(gate) * up for those 16 channels at column n/2.  It excludes the other steps. */
enum {
    B200FC_STEP_NONE = 0,
    B200FC_STEP_DEQUANT = 1,
    B200FC_STEP_BIAS = 2,
    B200FC_STEP_GELU = 4,
    B200FC_STEP_QUANT = 8,
    B200FC_STEP_SILU_MUL = 16
};

/* What PP::BiasGeluStore<D, steps> captures (include/kernels_amx.hpp:552-583), as plain data.  Arrays are indexed by
 * the GLOBAL output column n, as the reference functor is (kernels_amx.hpp:1250,1294). */
typedef struct {
    int steps;                     /* B200FC_STEP_* bitmask */
    int out_dtype;                 /* B200FC_F32 / B200FC_BF16 / B200FC_S8, or B200FC_S32 = raw int32 accumulators */
    void* C;                       /* output matrix [M, N] */
    int64_t ldc_bytes;
    const float* bias;             /* [N] fp32, needed with STEP_BIAS (set_bias, :560-563) */
    float deq_scale;               /* per-tensor dequant scale (set_deq_scale, :565-570) */
    const float* deq_scale_per_oc; /* optional [N]: extra per-output-channel dequant factor (no reference counterpart;
                                      needed for per-channel int8 weights) */
    float q_scale;                 /* per-tensor quant scale (set_q_scale(float), :572-577) */
    const float* q_scale_per_oc;   /* optional [N]: per-output-channel quant scale (set_q_scale(float*), :578-583) */
} b200fc_epilogue_t;

/* ---- library ---------------------------------------------------------------------------------------------- */
const char* b200fc_last_error(void);
const char* b200fc_version(void);
/* number of this library's kernels launched by the calling process so far (bench bookkeeping) */
int64_t b200fc_launch_count(void);

/* Limits the persistent GEMM kernels to `sms` SMs (0 = all).  A tensor-parallel caller that overlaps an NCCL
 * all-reduce with the GEMMs leaves the collective a few SMs this way; otherwise its CTAs queue behind the GEMM's. */
int b200fc_set_sm_limit(int sms);

/* CTAs per SM of the decode kernel (M <= 16): 2 (the default, 0 restores it) is fastest for a chain of dependent layers
 * on one stream; 1 lets two decode kernels of DIFFERENT streams be resident together, so that independent layers
 * overlap one another's ramp and tail (how the reference times its weight stream: L layers that share no data,
 * weight_compression/fc16m.cpp:687-734, main.cpp:811-846). */
int b200fc_set_decode_ctas_per_sm(int n);

/* waits for `stream` and reports whether any kernel of this library gave up on a bounded wait since the last check
 * (B200FC_ERR_KERNEL); the _host entry points do this themselves */
int b200fc_sync_check(void* stream);
/* Every wait inside a kernel (on a shared-memory barrier, on another GPU's arrival counter) is bounded; a wait that
 * runs out makes the kernel stop cleanly and b200fc_sync_check report B200FC_ERR_KERNEL.  Sets that bound for
 * kernels launched from now on (default 2 s; at least 1 us).  The reference has no counterpart (its only rendez-vous
 * is an atomic between two threads, tests/amx-mlp.cpp:656-660). */
int b200fc_set_wait_limit_ns(uint64_t ns);

/* ---- packed weights: the `internalB` cache of amx_kernel::Matmul (include/kernels_amx.hpp:1045-1072) ---------- */
typedef struct b200fc_weight b200fc_weight_t;

typedef enum {
    B200FC_PACK_PLAIN = 0,       /* keep the dtype of B (bf16 / s8 / u8): repackB_1x2, kernels_amx.hpp:761-816 */
    B200FC_PACK_QUANT_TENSOR = 1,/* bf16 B -> int8 with one absmax scale, the compressed-weight path
                                    Matmul<bf16,int8_t,float>, kernels_amx.hpp:1363-1377 */
    B200FC_PACK_INT8_CHANNEL = 2,/* s8 B + caller's per-output-channel fp32 scales [N] (no reference counterpart) */
    B200FC_PACK_INT4_GROUP = 3   /* bf16 B -> 4-bit values in [-7, 7] with one fp32 absmax scale per output channel and
                                    group of B200FC_INT4_GROUP consecutive K.  The reference reserves this precision
                                    (Weight_INT4, main.cpp:36) and measures its upper bound with a dequantisation that
                                    does no arithmetic (fake_dequant_i4_16x32, weight_compression/wcompress.hpp:122-134)
                                    but defines no algorithm; the scheme is the int8 one of kernels_amx.hpp:1363-1377
                                    per group: q = rne(w * (7 / absmax)), dequantised value = q * (absmax / 7). */
} b200fc_pack_mode_t;
#define B200FC_INT4_GROUP 128

/* Packs B once.  transposeB = 0: B is [K, N]; 1: B is [N, K] (Matmul ctor flag, kernels_amx.hpp:1071, getSubMatB
 * :699-705).  B may be a host or a device pointer.  `scales`: B200FC_PACK_INT8_CHANNEL needs the [N] per-channel
 * scales; B200FC_PACK_QUANT_TENSOR accepts an optional pointer to ONE float, the absmax to quantise with (the reference
 * takes the absmax of the whole B even when a thread packs only its column range, kernels_amx.hpp:1370); NULL = absmax
 * of the given matrix. */
int b200fc_weight_pack(const void* B, int dtypeB, int K, int N, int64_t ldb_bytes, int transposeB, int pack_mode,
                       const float* scales, b200fc_weight_t** out, void* stream);
int b200fc_weight_free(b200fc_weight_t* w);
/* K, N, dtype of the stored weights (B200FC_BF16/S8/U8), whether they are dequantised on the fly, tensor scale */
int b200fc_weight_info(const b200fc_weight_t* w, int* K, int* N, int* dtype, int* compressed, float* deq_scale);
/* copies the packed weights back as a plain row-major [N, K] matrix of their stored dtype (host or device dst);
 * 4-bit weights come back as one int8 per value */
int b200fc_weight_unpack(const b200fc_weight_t* w, void* dst, int64_t ld_bytes, void* stream);
/* the dequant scales of B200FC_PACK_INT4_GROUP weights as a row-major fp32 matrix [N, ceil(K / B200FC_INT4_GROUP)]
 * in HOST memory (ld_bytes >= 4 * groups); synchronises the stream */
int b200fc_weight_group_scales(const b200fc_weight_t* w, float* host_dst, int64_t ld_bytes, void* stream);

/* Serialised packed weights: a self-describing blob in HOST memory (64-byte header, the packed matrix as it lies in
 * HBM, then the per-channel scales if the object has them) that b200fc_weight_import turns back into an identical
 * object without re-packing or re-quantising.  The reference has no on-disk form — it re-packs at every start-up — but
 * its torch extension clones the packed copy in __deepcopy__ (torch-ext/amx_mlp.cpp:499-510); this pair serves both
 * uses (checkpoint files of packed weights, clones).  The blob is tied to this library's packing (version in the
 * header); import rejects anything else with B200FC_ERR_INVALID.  Both calls synchronise the stream. */
int b200fc_weight_export_size(const b200fc_weight_t* w, size_t* bytes);
int b200fc_weight_export(const b200fc_weight_t* w, void* host_dst, size_t capacity, void* stream);
int b200fc_weight_import(const void* host_src, size_t bytes, b200fc_weight_t** out, void* stream);

/* ---- Matmul::operator()(A, B, n0, n1, ppkernel), include/kernels_amx.hpp:1169-1314 and :1343-1516 ------------- */
/* C[:, n0:n1) = postops(A[M,K] * W[:, n0:n1)).  dtypeA: B200FC_BF16 with bf16 or compressed weights, B200FC_S8 /
 * B200FC_U8 with s8 / u8 weights.  With compressed weights STEP_DEQUANT is required and the weight's own scale(s)
 * replace ep->deq_scale, as the reference's set_deq_scale() call does (kernels_amx.hpp:1379).  4-bit weights: the
 * group scales are applied to the group sums inside the kernel, and n0 must be a multiple of 128. */
int b200fc_matmul(const b200fc_weight_t* W, const void* A, int dtypeA, int M, int K, int64_t lda_bytes, int n0, int n1,
                  const b200fc_epilogue_t* ep, void* stream);
/* Same call with A, ep->C, ep->bias and the per-channel scale arrays in HOST memory: stages them through device
 * buffers owned by the weight object, runs, copies C back and synchronises the stream (what a caller of the CPU
 * reference gets: results in host memory when the call returns). */
int b200fc_matmul_host(b200fc_weight_t* W, const void* A, int dtypeA, int M, int K, int64_t lda_bytes, int n0, int n1,
                       const b200fc_epilogue_t* ep, void* stream);

/* ---- MatmulVector::operator()(A, b, c) and GemAvB, include/kernels_amx.hpp:959-1042, 1529-1618 --------------- */
/* c[M] = A[M,K] * b[K]; dtype B200FC_BF16 -> fp32 c, B200FC_S8 -> int32 c.  Any K >= 1 (the reference limits K). */
int b200fc_matvec(const void* A, int dtype, int M, int K, int64_t lda_bytes, const void* b, void* c, void* stream);
int b200fc_matvec_host(const void* A, int dtype, int M, int K, int64_t lda_bytes, const void* b, void* c, void* stream);

/* ---- fused Llama MLP: AMX_MLP::MLP::setup / run, tests/amx-mlp.cpp:752-783 ----------------------------------- */
typedef struct b200fc_mlp b200fc_mlp_t;
/* gate, up: [N, K]; down: [K, N]; bf16, contiguous, torch nn.Linear layout (host or device pointers).
 * tp_size > 1 keeps only this rank's Megatron shard: rows [rank*N/tp, (rank+1)*N/tp) of gate and up and the same
 * columns of down; b200fc_mlp_run_partial then yields the rank's fp32 contribution to the output.
 * Requirements: K % 64 == 0, (N / tp_size) % 32 == 0 (the reference needs N % 32 == 0, K % 256 == 0, :552-553). */
int b200fc_mlp_create(const void* gate, const void* up, const void* down, int K, int N, int tp_rank, int tp_size,
                      b200fc_mlp_t** out, void* stream);
int b200fc_mlp_free(b200fc_mlp_t* mlp);
/* grows the internal activation buffer for up to max_M rows (the reference's actUp grows inside run, :771-776) */
int b200fc_mlp_reserve(b200fc_mlp_t* mlp, int max_M);
/* out[M,K] bf16 = down(silu(x gate^T) * (x up^T)); x [M,K] bf16.  tp_size must be 1. */
int b200fc_mlp_run(b200fc_mlp_t* mlp, const void* x, int64_t ldx_bytes, int M, void* out, int64_t ldo_bytes,
                   void* stream);
/* this rank's contribution to the output, [M,K] in out_dtype B200FC_F32 or B200FC_BF16; the caller sums it over
 * ranks (one all-reduce) and, for fp32, rounds to bf16 (the reference rounds after the fp32 sum, :672-680) */
int b200fc_mlp_run_partial(b200fc_mlp_t* mlp, const void* x, int64_t ldx_bytes, int M, void* partial, int out_dtype,
                           int64_t ldp_bytes, void* stream);
/* The two stages on their own, as the reference exposes them (Linear::runGateUp, tests/amx-mlp.cpp:707-737, and
 * Linear::run, :648-704): gate_up writes the internal [M, N/tp] bf16 activation, down consumes it. */
int b200fc_mlp_gate_up(b200fc_mlp_t* mlp, const void* x, int64_t ldx_bytes, int M, void* stream);
int b200fc_mlp_down(b200fc_mlp_t* mlp, int M, void* out, int out_dtype, int64_t ldo_bytes, void* stream);
/* Linear::run on a row range: rows [row0, row0 + rows) of the activation left by the last b200fc_mlp_gate_up ->
 * out[rows, K] (out points at the first of those rows).  Lets a tensor-parallel caller reduce finished row blocks
 * while the following ones are still being multiplied. */
int b200fc_mlp_down_rows(b200fc_mlp_t* mlp, int row0, int rows, void* out, int out_dtype, int64_t ldo_bytes, void* stream);
/* Down projection fused with the tensor-parallel all-reduce (no reference counterpart; the reference's pairwise
 * split-K reduce, tests/amx-mlp.cpp:656-683, is its single-process ancestor).  `multicast_out` is an NVLink
 * multicast (NVLS) mapping of the [M, K] output that every rank of the group has bound, e.g. the multicast_ptr of a
 * torch symmetric-memory buffer; the GEMM epilogue adds this rank's contribution into ALL replicas with
 * multimem.red, so no separate collective runs.  The caller zeroes the replicas and separates steps with a
 * cross-rank barrier (see mm_amx_b200/tp.py).  Needs M > 16; split-K shapes are not supported. */
int b200fc_mlp_down_reduce(b200fc_mlp_t* mlp, int M, void* multicast_out, int out_dtype, int64_t ldo_bytes, void* stream);
/* Down projection with the tensor-parallel all-reduce done by the same kernel, pull style (no reference
 * counterpart).  Three symmetric buffers are shared by the ranks of the group (e.g. torch symmetric memory):
 * `partial` and `out`, both [>= M, K] bf16 with row pitch ld_bytes, each also mapped through an NVLink multicast
 * address, and one array of 32-bit arrival counters per rank.  Most CTA pairs multiply and store this rank's tile
 * into its `partial` replica, then bump the tile's counter on the tile's owner (tile index % world); the last
 * `comm_sms` SMs of the grid (and every other SM once its tiles are done) wait for the tiles this rank owns, pull
 * them from all replicas with multimem.ld_reduce (summed in the switch, fp32 accumulation) and write the sum to
 * every rank's `out` with multimem.st.  Each contribution crosses NVLink once and the transfer overlaps the multiplication of later tiles.
 * Contract: the counters the call uses are zero when it starts on any rank; after the call every rank passes a
 * cross-rank barrier before `out` is read, `partial` is rewritten or the counters are cleared (mm_amx_b200/tp.py
 * alternates two counter arrays so that one barrier per step suffices).  Needs M > 16, K % 8 == 0, 2 <= world <= 8,
 * and a GPU not shared with other kernels (the whole grid must be resident).  Waits are bounded (B200FC_ERR_KERNEL
 * at the next b200fc_sync_check). */
typedef struct {
    int world, rank;
    void* partial_local;     /* this rank's replica of `partial` */
    const void* partial_mc;  /* multicast address of `partial` */
    void* out_mc;            /* multicast address of `out` */
    int64_t ld_bytes;
    uint32_t* flags[8];      /* flags[r]: counter array of rank r as mapped on this GPU */
    int max_tiles;           /* entries per counter array; a call uses 2 * ceil(M/256) * ceil(K/256) of them and the last one (hands out reduction work) */
    int comm_sms;            /* SMs that reduce instead of multiplying from the start (even; 8 measured best at 8 GPUs) */
} b200fc_allreduce_t;
int b200fc_mlp_down_allreduce(b200fc_mlp_t* mlp, int M, const b200fc_allreduce_t* ar, void* stream);
/* x and out in HOST memory; copies, runs, copies back, synchronises.  From M = 512 on the rows flow through a
 * copy-in / compute / copy-out pipeline over three internal streams (short row chunks first and last, so that little of
 * the PCIe time is exposed), which needs pinned host buffers to overlap; results per row are those of b200fc_mlp_run up
 * to the last bit of a bf16 (a short chunk may take the K-split route of the GEMM, which adds in another order). */
int b200fc_mlp_run_host(b200fc_mlp_t* mlp, const void* x, int64_t ldx_bytes, int M, void* out, int64_t ldo_bytes,
                        void* stream);
/* How b200fc_mlp_run_host cuts a batch of M rows of an MLP with hidden size K and intermediate size N: rows per
 * gate/up launch (each preceded by the copy-in of its rows) and rows per down launch (each followed by the copy-out of
 * its rows); both lists sum to M.  A pure host function (no reference counterpart: AMX_MLP::MLP::run works in place in
 * host memory, tests/amx-mlp.cpp:778-783); `capacity` = entries each array can take. */
int b200fc_mlp_host_plan(int M, int K, int N, int* gate_up_rows, int* down_rows, int capacity, int* n_gate_up, int* n_down);
/* The same forward for decode-shaped batches (1 <= M <= 16) WITHOUT any allocation — no counterpart in the
 * reference.  For callers that may not enter the CUDA allocator while they run (a serving loop with a frozen memory
 * plan, code that must not trigger the device synchronisation cudaMalloc / cudaFree imply).  The gate/up activation
 * lives in a fixed 1 MiB device array inside the library image, so M * (N / tp) * 2 bytes must not exceed
 * b200fc_mlp_decode_static_capacity(); larger requests fail with B200FC_ERR_INVALID.  A second fixed array (about
 * 5 MiB) holds the decode kernel's partial sums and arrival counters; b200fc_mlp_decode_static_footprint() is the total
 * every GPU that loads the library holds until the process exits.  out is [M, K] in out_dtype B200FC_BF16 (the full
 * result when tp_size == 1) or B200FC_F32 / B200FC_BF16 (this rank's contribution otherwise).
 *   - The first call on each device looks up the device addresses of these arrays and of the library's status word
 *     (all three are part of the image: nothing is allocated) and sets the kernels' shared-memory attribute; make
 *     that first call during start-up, before any stream capture begins.
 *   - All calls on a device share the arrays: calls whose kernels can overlap on the GPU (different streams
 *     without ordering) race on them.  Calls on one stream are ordered and safe.
 *   - The arrays keep the previous call's contents; every element a call reads it has written first, and the
 *     counters are back at zero when a call's kernels finish. */
int b200fc_mlp_run_decode_static(b200fc_mlp_t* mlp, const void* x, int64_t ldx_bytes, int M, void* out, int out_dtype,
                                 int64_t ldo_bytes, void* stream);
int64_t b200fc_mlp_decode_static_capacity(void);
int64_t b200fc_mlp_decode_static_footprint(void);
/* ---- the steps either side of the MLP in a Llama block -------------------------------------------------------------- */
/* out[M,K] bf16 = RMSNorm(x): y = x * rsqrt(mean(x^2) + eps) in fp32, rounded to bf16 — the weight-less LlamaRMSNorm
 * the reference's benchmark script puts in front of every MLP (torch-ext/test.py:161-176).  `weight` (bf16 [K], may be
 * NULL) multiplies the rounded value, rounded again (the form with a learned scale). */
int b200fc_rmsnorm(const void* x, int64_t ldx_bytes, int M, int K, const void* weight, float eps, void* out,
                   int64_t ldo_bytes, void* stream);
/* One MLP block of a Llama layer: out = (add_residual ? x : 0) + MLP(RMSNorm(x)).  The reference chains
 * LlamaRMSNorm -> MLP per layer (torch-ext/test.py:178-189); the residual add has no reference counterpart.  The
 * normalisation is one small kernel ahead of gate/up; the residual is added in the down projection's epilogue, in fp32,
 * before the single bf16 rounding of the output.  tp_size must be 1; out must not alias x. */
int b200fc_mlp_run_block(b200fc_mlp_t* mlp, const void* x, int64_t ldx_bytes, int M, float eps, const void* norm_weight,
                         int add_residual, void* out, int64_t ldo_bytes, void* stream);
/* device pointer to the [M, N/tp] bf16 activation of the last run (debug / layer-wise parity) */
const void* b200fc_mlp_act(const b200fc_mlp_t* mlp);

/* ---- decode attention: one query token per sequence against a bf16 key/value cache --------------------------------- */
/* out[b, h, :] = sum_n softmax_n(scale * q[b, h, :] . k[b, h / G, n, :]) * v[b, h / G, n, :],  n < len(b),  G = H / Hkv.
 * The reference's pieces grown into one kernel: w = query x Key^T on the AMX unit (MatMulVec_AMX, test_jit.cpp:17-95;
 * MatmulVector, include/kernels_amx.hpp:959-1042) and the one-token attention that cuts the key range into blocks,
 * encodes each into a sub-state (score maximum, sum of exponentials, weighted values) and combines the sub-states
 * (MHA2Kernels, include/kernels_mha.hpp:146-270: fp32, q {B,1,H,K}, k and v {B,H,N,K}, softmax without a scale
 * factor — pass scale = 1 for that).  Here q, k, v are bf16, the softmax runs in fp32, G query heads may share one kv
 * head (G <= 16; the reference has G = 1), sequences may have their own lengths, and all strides are explicit.
 * D must be 64 or 128; k, v and their strides 16-byte aligned.  A sequence of length 0 yields zeros. */
typedef struct {
    int B, H, Hkv, N, D;            /* sequences, query heads, kv heads, cache length (tokens), head size */
    const void* q;                  /* [B, H, D] bf16 */
    int64_t q_batch_stride, q_head_stride;                 /* bytes */
    const void* k; const void* v;   /* [B, Hkv, N, D] bf16 each */
    int64_t kv_batch_stride, kv_head_stride, kv_token_stride;   /* bytes, the same for k and v */
    void* out;                      /* [B, H, D] in out_dtype (B200FC_BF16 or B200FC_F32) */
    int64_t out_batch_stride, out_head_stride;
    int out_dtype;
    const int32_t* seq_lens;        /* optional device array [B]: tokens of sequence b (clamped to [0, N]); NULL = N */
    float scale;
} b200fc_attention_t;
int b200fc_decode_attention(const b200fc_attention_t* a, void* stream);

/* ---- device memory for callers that do not link the CUDA runtime themselves ------------------------------------ */
int b200fc_device_malloc(void** ptr, int64_t bytes);
int b200fc_device_free(void* ptr);
/* copy between any two of host / device memory (direction inferred), ordered on `stream`, then waits for it */
int b200fc_memcpy(void* dst, const void* src, int64_t bytes, void* stream);

/* ---- helpers -------------------------------------------------------------------------------------------------- */
/* bf16 round-to-nearest-even of fp32 on the device: out[i] = bf16(a[i] + (b ? b[i] : 0)) */
int b200fc_add_round_bf16(const float* a, const float* b, void* out_bf16, int64_t n, void* stream);
/* writes `bytes` bytes of a scratch buffer larger than L2 so that the next kernel starts cache-cold
 * (the role of the reference's clflush helper, torch-ext/amx_mlp.cpp:514-522) */
int b200fc_flush_l2(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200FC_H */
