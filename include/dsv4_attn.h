/*
 * dsv4_attn.h - C ABI of the B200 (sm_100a) decode-attention library for
 * DeepSeek-V4-style attention: CSA sparse decode, HCA dense decode, and the
 * split-KV merge.
 *
 * Conventions (the same ones the reference project's C entry point follows,
 * hca/sm100/kernel.cu:269-358):
 *   - every pointer is a raw DEVICE pointer owned by the caller; the library
 *     allocates nothing.  State kept between calls: per-device "attribute set"
 *     flags and the address of the built-in scratch array of
 *     dsv4_csa_sparse_decode_fwd_noalloc (each written once), and the test
 *     switches at the end of this file.  The 32 MiB scratch array is part of the
 *     library image: every GPU context that loads the library holds it, whether or
 *     not that entry point is ever called;
 *   - work is enqueued on the `stream` argument (a cudaStream_t passed as
 *     void*, NULL = default stream) and the call returns without synchronising;
 *   - the return value is 0 on success, otherwise a cudaError_t value
 *     (cudaErrorInvalidValue = 1 for rejected arguments).  Nothing throws and
 *     nothing aborts.
 *
 * Cache entry (the packed 656-byte layout), 16-byte aligned:
 *     [  0,512)  512 x FP8 e4m3 latent (also the value vector, d_v = 512)
 *     [512,528)  4 x FP32 scale, one per 128 latent elements (value = fp8*scale)
 *     [528,656)  64 x BF16 RoPE tail (already rotated)
 * A page is 64 consecutive entries (41,984 bytes).  A pool is an array of
 * pages; a request's block table maps logical page number -> pool page.
 */
#ifndef DSV4_ATTN_H_
#define DSV4_ATTN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DSV4_D_LATENT      512
#define DSV4_D_ROPE        64
#define DSV4_D_QK          576
#define DSV4_D_V           512
#define DSV4_ENTRY_BYTES   656
#define DSV4_PAGE_ENTRIES  64
#define DSV4_MAX_SPLITS    64

/* Words of the optional `status` array a kernel writes when one of its bounded
 * waits gives up (it never traps and never spins without limit), or when an index,
 * a length or a block-table value points outside the cache (code 7: the entry is
 * left out of the softmax and nothing is read through it).  When status[0] != 0
 * after a call, `out` and `lse` of that call are undefined: pass `status` wherever
 * the inputs are not trusted. */
#define DSV4_STATUS_WORDS  4   /* [0] error code (0 = none), [1] block x|y<<8|z<<20, [2] role, [3] tile or entry */
#define DSV4_STATUS_BAD_INDEX 7

/*
 * CSA sparse decode.  For each request b and query token j the kernel gathers
 * the cache entries named by indices[b][j][0..topk) through block_table[b],
 * and computes softmax(q . k^T * sm_scale) . v over them in one pass.
 *
 * Takes the place of the reference's gather + attention core on pre-projected
 * tensors (bench/bench/reference.py:576-580 followed by :516-545); the
 * parameter-struct style follows hca/params.h:10-77 and csa/params.h:12-39.
 * Arithmetic: FP32 accumulation; Q, P and the dequantised entries pass through FP16 operands.
 * PRECONDITIONS of that operand type (both packed-layout entry points): |q| < 65504, and block
 * scales <= 146 - a block with a larger scale (entries beyond +-65408) is clamped to 146.  Inputs
 * of the N(0,1) kind the cache is built for are far inside both; dsv4_attn_b200.api offers a
 * host-side check (check_fp16_range=True) for callers that cannot vouch for theirs.
 */
typedef struct Dsv4CsaSparseDecodeParams {
    int32_t B;                  /* requests */
    int32_t s_q;                /* query tokens per request (1, or 2 for speculative decode) */
    int32_t H;                  /* query heads */
    int32_t topk;               /* length of each index list */
    int32_t max_pages;          /* row length of block_table */
    int32_t num_splits;         /* >= 1; > 1 needs partial_o / partial_lse */
    float   sm_scale;           /* softmax scale, usually 1/sqrt(576) */
    int32_t reserved0;
    int64_t num_pages;          /* pages in kv_pool: block-table values outside [0, num_pages) are not followed (status code 7) */
    const void*    q;           /* bf16  [B, s_q, H, 576] */
    const void*    kv_pool;     /* uint8 [num_pages, 64, 656] */
    const int32_t* block_table; /* int32 [B, max_pages] */
    const int32_t* indices;     /* int32 [B, s_q, topk]; negative = padding */
    const int32_t* kv_len;      /* optional int32 [B, s_q]: indices >= kv_len are masked (causality
                                   between speculative tokens); NULL = no bound */
    const int32_t* topk_len;    /* optional int32 [B, s_q]: only the first topk_len slots of each index list
                                   are read (ragged batches padded to a common topk); NULL = all topk */
    const float*   attn_sink;   /* optional float [H], natural-log units, added to the denominator */
    void*          out;         /* bf16  [B, s_q, H, 512] */
    float*         lse;         /* optional float [B, s_q, H], natural log, sink excluded, -inf if empty */
    float*         partial_o;   /* scratch of num_splits*B*s_q*H*512 floats when num_splits > 1 (contents unspecified afterwards) */
    float*         partial_lse; /* float [num_splits, B*s_q, H], log2 units */
    int32_t*       status;      /* optional int32 [DSV4_STATUS_WORDS], zeroed by the caller */
    const void*    sched;       /* optional plan written by dsv4_attn_plan for this batch (kind CSA, same B, s_q, H and
                                   lengths): num_splits is then ignored and partial_o / partial_lse must have the sizes
                                   dsv4_attn_sched_bytes reports */
} Dsv4CsaSparseDecodeParams;

int dsv4_csa_sparse_decode_fwd(const Dsv4CsaSparseDecodeParams* p, void* stream);

/*
 * CSA sparse decode for callers that cannot allocate device memory.  No
 * counterpart in the reference.
 *
 * Some hosts of this library cannot call cudaMalloc at the point where they
 * decode: a serving engine that has handed all of HBM to its KV-cache pool, a
 * plug-in loaded into a process whose allocator it must not touch, code running
 * inside a region where allocation is forbidden.  With num_splits > 1 the
 * ordinary entry point needs a caller-provided workspace for the split
 * partials; this one keeps that workspace inside the library image instead: a
 * fixed device array of 32 MiB (+ 64 KiB for the partial LSEs) that every GPU
 * loading the library holds until the process exits.  p->partial_o and
 * p->partial_lse are ignored; everything else means what it means for
 * dsv4_csa_sparse_decode_fwd, and the results are identical.
 *
 * Limit: num_splits * B * s_q * H * 512 <= 8 Mi floats (for example 8 splits
 * of 16 rows of 128 heads).  Larger requests are rejected with
 * cudaErrorInvalidValue before anything is enqueued, and
 * dsv4_attn_last_error() says why.  The call itself allocates nothing and frees
 * nothing.
 *
 * The first call on a device looks the array's device address up (once per
 * device, with that device current); make that first call outside any stream
 * capture.  All calls share the one array: the decode kernel overwrites every
 * partial the merge reads, so nothing has to be cleared between calls, but two
 * calls that overlap on the GPU (different streams) race on it - serialise them.
 */
int dsv4_csa_sparse_decode_fwd_noalloc(const Dsv4CsaSparseDecodeParams* p, void* stream);

/* Size in bytes of the built-in scratch used by the entry point above. */
int64_t dsv4_noalloc_scratch_bytes(void);

/* Why the calling thread's last call to an entry point that sets it was rejected ("" if it was not). */
const char* dsv4_attn_last_error(void);

/*
 * HCA dense decode.  Query token j of request b attends to every compressed
 * entry [0, kv_len[b][j]) of the request (through the block table) followed by
 * the first win_len[b][j] rows of the request's sliding-window buffer, in one
 * softmax.
 *
 * Takes the place of the reference's hca_decode_forward
 * (bench/bench/reference.py:471-546) and of its kernel parameter block
 * (hca/params.h:10-77), with per-request lengths instead of one M_cur/swa_len
 * for the whole batch.
 */
typedef struct Dsv4HcaDenseDecodeParams {
    int32_t B;
    int32_t s_q;
    int32_t H;
    int32_t max_pages;
    int32_t win_cap;            /* rows per request in win_pool (W, usually 128) */
    int32_t num_splits;
    float   sm_scale;
    int32_t reserved0;
    int64_t num_pages;
    const void*    q;           /* bf16  [B, s_q, H, 576] */
    const void*    kv_pool;     /* uint8 [num_pages, 64, 656] */
    const int32_t* block_table; /* int32 [B, max_pages] */
    const int32_t* kv_len;      /* int32 [B, s_q] compressed entries visible to each query token */
    const void*    win_pool;    /* uint8 [B, win_cap, 656] */
    const int32_t* win_len;     /* int32 [B, s_q] window rows visible to each query token */
    const float*   attn_sink;   /* optional float [H] */
    void*          out;         /* bf16  [B, s_q, H, 512] */
    float*         lse;         /* optional float [B, s_q, H] */
    float*         partial_o;
    float*         partial_lse;
    int32_t*       status;
    const void*    sched;       /* optional plan (kind HCA), as in Dsv4CsaSparseDecodeParams */
} Dsv4HcaDenseDecodeParams;

int dsv4_hca_dense_decode_fwd(const Dsv4HcaDenseDecodeParams* p, void* stream);

/*
 * LSE-weighted merge of split-KV partials.  Same algebra and the same field
 * meaning as the reference's HcaCombineParams / launch_hca_combine
 * (hca/sm100/combine.h:9-31, hca/sm100/combine.cu:25-145); `N` is the
 * reference's B times the number of query tokens, and strides are in elements.
 */
typedef struct Dsv4CombineParams {
    int32_t N;                  /* rows = B * s_q */
    int32_t H;
    int32_t D;                  /* must be 512 */
    int32_t num_splits;         /* 1 .. 1024 */
    const float* partial_o;     /* [split, N, H, D] */
    const float* partial_lse;   /* [split, N, H], log2 units, -inf = empty split */
    void*        out;           /* bf16 [N, H, D] */
    float*       lse;           /* optional [N, H], natural log */
    const float* attn_sink;     /* optional [H], natural-log units */
    int64_t stride_po_split, stride_po_n, stride_po_h;
    int64_t stride_pl_split, stride_pl_n;
    int64_t stride_out_n, stride_out_h;
    int64_t stride_lse_n;
} Dsv4CombineParams;

int dsv4_attn_combine(const Dsv4CombineParams* p, void* stream);

/*
 * Split-KV planning (host arithmetic only, safe during stream capture).
 * Chooses how many splits each (request, query token) should use so that the
 * grid fills `num_sms` SMs without excess partial traffic.  The reference's
 * counterpart is the static one-tile-per-split rule of
 * hca/sm100/helpers.h:831-869 and hca/sm100/kernel.cu:248-257.
 *   rows      = B * s_q
 *   H         = query heads
 *   max_len   = longest per-row entry count (topk for CSA, kv_len+win_len for HCA)
 *   num_sms   = 0 -> query the current device
 * Returns the split count (>= 1, <= DSV4_MAX_SPLITS), or a negative cudaError_t.
 */
int dsv4_attn_plan_splits(int rows, int H, int max_len, int num_sms);

/* Bytes of partial_o + partial_lse a call with these sizes needs (0 when
 * num_splits == 1).  partial_lse starts at the returned `*lse_offset`. */
int64_t dsv4_attn_workspace_bytes(int rows, int H, int num_splits, int64_t* lse_offset);

/*
 * Split-KV scheduler.  dsv4_attn_plan launches a small planner kernel (one block; no host
 * synchronisation, no allocation, capturable into a CUDA graph) that reads the per-row lengths
 * of a batch and writes a work list into `sched`: every (row, group of 128 heads) is cut into
 * items of 64-entry tiles so that the SMs of the device get equal shares of tiles plus per-item
 * set-up; a row that fits one share is written out directly, a row that straddles shares gets
 * partial slots that the merge adds up.  The decode entry points given that `sched` then run as
 * resident blocks (two per pair of SMs, one half of the value columns each) that walk their share
 * of the list, keep tensor memory and barriers alive between items and fetch the next item's
 * queries and first tiles while the current one finishes.  A plan depends only on B, s_q, H and
 * the length arrays, so one plan serves every layer of a decode step that shares them.
 * num_splits = 0 lets the planner balance; num_splits >= 1 cuts every unit into that many equal
 * pieces (what a caller that fixes the split count asks for) and deals the pieces out in order;
 * consecutive pieces of a unit that fall to the same pair of SMs run there as one item (their
 * partial results would only be added up again), so a unit ends up with at most num_splits items.
 * Replaces the reference's static one-tile-per-split rule (hca/sm100/helpers.h:831-869,
 * hca/sm100/kernel.cu:99-102,248-257).
 *
 * dsv4_attn_sched_bytes: size of `sched` for a shape, and the sizes of the partial_o (BF16 slots)
 * and partial_lse areas the decode call then needs.  num_sms = 0 -> the current device.
 */
#define DSV4_PLAN_CSA 0
#define DSV4_PLAN_HCA 1
typedef struct Dsv4PlanParams {
    int32_t kind;               /* DSV4_PLAN_CSA or DSV4_PLAN_HCA */
    int32_t B;
    int32_t s_q;
    int32_t H;
    int32_t topk;               /* CSA: length of each index list */
    int32_t num_splits;         /* 0 = balance over the SMs, >= 1 = that many pieces per unit (see above) */
    int32_t num_sms;            /* 0 = all SMs of the current device (fewer may be given, never more) */
    int32_t reserved0;
    const int32_t* topk_len;    /* CSA, optional int32 [B, s_q] */
    const int32_t* kv_len;      /* HCA int32 [B, s_q]; CSA: optional, passed through to the items */
    const int32_t* win_len;     /* HCA int32 [B, s_q] */
    void*   sched;              /* device buffer, 16-byte aligned */
    int64_t sched_bytes;
} Dsv4PlanParams;

int64_t dsv4_attn_sched_bytes(int rows, int H, int num_splits, int num_sms, int64_t* partial_o_bytes,
                              int64_t* partial_lse_bytes);
int dsv4_attn_plan(const Dsv4PlanParams* p, void* stream);

/* The same plan computed serially on the host: every pointer of `p` (length arrays and `sched`) is then a
 * HOST pointer and num_sms must be given (> 0; no device is asked).  For inspecting what the planner does
 * and for testing its arithmetic without a GPU - the decode entry points take device plans only.  Items of
 * one block pair may come in another order than from the kernel.  Layout of the buffer in int32 words:
 * [0,16) info (items, partial slots, 1 = capacity exceeded, cost share per pair); [16, 16+1025) first item of
 * every pair; then, each padded to 4 words, pieces per unit and first slot per unit (units = rows x head
 * groups); a 64-bit scratch word per unit (padded to an even count); then the items, 8 words each: row, head
 * group, first tile, tiles, partial slot (-1 = writes the final output), entries of the row, the row's second
 * length (CSA: causal bound; HCA: compressed entries), 0. */
int dsv4_attn_plan_host(const Dsv4PlanParams* p);

/*
 * The reference's entry point, kept symbol- and argument-compatible
 * (hca/sm100/kernel.cu:269-280; ctypes binding in
 * bench/bench/candidates/hca_custom_decode.py:60-73).  Reference cache layout:
 * Kc/Kswa uint8(e4m3) [B, M, 448], Kc_s/Kswa_s uint8(UE8M0) [B, M, 7],
 * Kc_rope/Kswa_rope bf16 [B, M, 64]; Q and O bf16 [B, n_h, 512]; the value
 * vector is the whole 512-wide row.  partial_O / partial_lse are workspaces
 * the caller sizes for (M_cur+swa_len)/128 splits; this library uses at most
 * that many.  Accepts any M_cur+swa_len >= 1 and any n_h >= 1 (a superset of
 * the reference's shape guard); still requires c == 448 and n_rope == 64.
 */
int hca_decode_fwd(const void* Q,
                   const void* Kc, const void* Kc_s, const void* Kc_rope,
                   const void* Kswa, const void* Kswa_s, const void* Kswa_rope,
                   const void* sink_logits,
                   void* O, void* partial_O, void* partial_lse,
                   float sm_scale,
                   int B, int n_h, int c, int n_rope,
                   int M_cur, int swa_len,
                   void* stream);

/*
 * CSA compressor, second pass (the cache-write side of the sparse path): for
 * every output block and channel a softmax over 2m gating logits - m own rows
 * (a-side) and the m rows of the previous block (b-side), each plus a
 * per-position bias - weights the 2m value rows; block 0 has no b-side.
 * Field for field the reference's CsaCompressReduceParams (csa/params.h:12-39)
 * behind the reference's csa_compress_reduce_fwd (csa/interface.h:21-85,
 * kernel csa/sm100/kernel.cuh:25-102), with 64-bit strides and the output
 * supplied by the caller.  All tensors BF16, strides in elements.  Returns
 * cudaErrorNotSupported for m != 4 (the reference instantiates only m = 4).
 */
typedef struct Dsv4CsaCompressReduceParams {
    int32_t B;              /* batch */
    int32_t n;              /* sequence length, divisible by m */
    int32_t c_out;          /* channels */
    int32_t m;              /* compression rate */
    const void* C_a;        /* bf16 [B, n, c_out] */
    const void* C_b;
    const void* Z_a;
    const void* Z_b;
    const void* B_a;        /* bf16 [m, c_out] */
    const void* B_b;
    void*       out;        /* bf16 [B, n/m, c_out] */
    int64_t stride_C_b;     /* batch stride of the four input streams */
    int64_t stride_C_n;     /* row stride of the four input streams */
    int64_t stride_out_b;
    int64_t stride_out_blk;
} Dsv4CsaCompressReduceParams;

int dsv4_csa_compress_reduce_fwd(const Dsv4CsaCompressReduceParams* p, void* stream);

/*
 * CSA indexer for decode (the step before the sparse decode): for every query token the
 * top-k visible compressed entries by
 *     score[t, s] = sum_h w[t, h] * relu(q[t, h, :] . k[s, :])
 * - the scoring and selection of the reference's lightning_indexer_topk after its
 * projections (bench/bench/reference.py:193-204; causal rule :197-201 expressed as
 * n_vis[t] = number of entries token t may see).  64 indexer heads of 128 dimensions.
 * Queries and keys are FP8 e4m3: q_fp8 [B, s_q, 64, 128] with the per-(token, head)
 * dequantisation scale folded by the caller into q_weight [B, s_q, 64] (= w * q_scale);
 * keys in pages of 64: 64 x 128 e4m3 bytes followed by the 64 FP32 scales of those keys
 * (8448 bytes per page), addressed through block_table [B, max_pages].  The FP8 x FP8
 * products are exact and accumulate in FP32 on the tensor cores.
 * Output: out_indices int32 [B, s_q, k], the k best entries in no particular order, -1
 * padded when fewer than k are visible; entries of equal score at the cut are chosen
 * arbitrarily.  `scores` is a caller-provided workspace, float [B*s_q, score_stride],
 * score_stride >= max_pages*64, holding the scores of the visible entries afterwards.
 * s_q is 1 or 2.  Pages the block table does not map into the pool score -inf.
 */
typedef struct Dsv4IndexerTopkParams {
    int32_t B;
    int32_t s_q;
    int32_t max_pages;
    int32_t k;
    int64_t num_pages;
    int64_t score_stride;
    const void*    q_fp8;        /* uint8 [B, s_q, 64, 128], 128-byte aligned */
    const float*   q_weight;     /* float [B, s_q, 64] */
    const void*    key_pages;    /* uint8 [num_pages, 8448], 128-byte aligned */
    const int32_t* block_table;  /* int32 [B, max_pages] */
    const int32_t* n_vis;        /* int32 [B, s_q] */
    float*         scores;       /* float [B*s_q, score_stride] workspace / optional result */
    int32_t*       out_indices;  /* int32 [B, s_q, k] */
    int32_t*       status;       /* optional int32[4], zeroed by the caller */
} Dsv4IndexerTopkParams;

int dsv4_indexer_topk_fwd(const Dsv4IndexerTopkParams* p, void* stream);

/*
 * Pre- and post-pass around the attention: partial RoPE on the last n_rope dimensions
 * of each vector (split-halves pairing, frequencies 1 / theta^(2i / n_rope); the
 * reference's apply_rope, bench/bench/reference.py:35-65), then - when norm_weight
 * is given - an RMS norm over the whole vector (rms_norm, reference.py:68-70), in
 * the order the reference's attention applies them to queries and keys
 * (reference.py:281-287).  inverse = 1 rotates by -position: the inverse RoPE the
 * reference applies to the attention output (reference.py:308-309), normally with
 * norm_weight = NULL.  x and out BF16 [n_rows, vecs_per_row, c] contiguous (out may
 * alias x); all vecs_per_row vectors of a row (the heads of a query token) share
 * positions[row].  n_rope = 64; c - 64 a multiple of 8, at most 512.
 */
typedef struct Dsv4RopeNormParams {
    int64_t n_rows;
    int32_t vecs_per_row;
    int32_t c;
    int32_t n_rope;
    int32_t inverse;
    float   eps;
    float   theta;              /* 10000 in the reference */
    const void*    x;
    void*          out;
    const int32_t* positions;   /* int32 [n_rows] */
    const void*    norm_weight; /* bf16 [c] or NULL */
} Dsv4RopeNormParams;

int dsv4_rope_norm_fwd(const Dsv4RopeNormParams* p, void* stream);

/*
 * HCA dense decode over a serving engine's packed cache pages, read in place, with
 * per-request lengths.  The bytes are the reference cache's (448 e4m3 latent with one
 * UE8M0 scale byte per 64 elements, 64 BF16 RoPE values; hca/params.h:27-46), laid out
 * as the engine stores them (hca/fixes.txt:79-101): a page of page_size tokens is
 *     [0, page_size*576)                 per token: 448 latent bytes | 128 RoPE bytes
 *     [page_size*576, page_size*584)     per token: 7 scale bytes | 1 pad byte
 * Token t of request b lives in page block_table[b][t / page_size], slot t % page_size.
 * Request b attends to its first m_cur[b] compressed tokens and the first swa_len[b]
 * tokens of its sliding-window pages, in one softmax (the per-request lengths asked for
 * in traces/hca_vs_sglang_sigs.txt:170-176, where the reference has one scalar for the
 * batch).  Q/O BF16 [B, H, 512]; the value row is the whole 512-wide row, the sink
 * enters the denominator only, as in hca_decode_fwd.  page_size 16, 32 or 64; pools
 * 64-byte aligned.  Either pool may be NULL if its lengths are all zero.
 */
typedef struct Dsv4HcaPackedDecodeParams {
    int32_t B;
    int32_t H;
    int32_t page_size;
    int32_t max_pages;          /* columns of block_table */
    int32_t swa_max_pages;      /* columns of swa_block_table */
    int32_t num_splits;         /* >= 1 */
    float   sm_scale;
    int32_t reserved0;
    int64_t num_pages;          /* pages in kv_pages (bounds are the caller's responsibility) */
    int64_t swa_num_pages;
    const void*    q;               /* bf16 [B, H, 512] */
    const void*    kv_pages;        /* uint8 [num_pages, page_size * 584] */
    const int32_t* block_table;     /* int32 [B, max_pages] */
    const int32_t* m_cur;           /* int32 [B] */
    const void*    swa_pages;       /* uint8 [swa_num_pages, page_size * 584] */
    const int32_t* swa_block_table; /* int32 [B, swa_max_pages] */
    const int32_t* swa_len;         /* int32 [B] */
    const float*   attn_sink;       /* float [H] natural-log units, or NULL */
    void*          out;             /* bf16 [B, H, 512] */
    float*         lse;             /* float [B, H] natural log, or NULL */
    float*         partial_o;       /* scratch of num_splits*B*H*512 floats when num_splits > 1 (contents unspecified afterwards) */
    float*         partial_lse;     /* float [num_splits, B, H] */
    int32_t*       status;          /* optional int32[4], zeroed by the caller */
} Dsv4HcaPackedDecodeParams;

int dsv4_hca_packed_decode_fwd(const Dsv4HcaPackedDecodeParams* p, void* stream);

/*
 * Destination of a cache insert: the paged pool of 656-byte entries and, per
 * request, the logical index of the first entry to write (normally the number of
 * entries the request already has).  Entry e of request b goes to page
 * block_table[b][e / 64], slot e % 64.  A position outside the block table, or a
 * table value outside the pool, is skipped and reported through `status`
 * (status[0] = 16, status[1] = request, status[2] = position) - nothing is
 * written out of bounds.  Paging has no counterpart in the reference.
 */
typedef struct Dsv4CacheDest {
    void*          kv_pool;      /* uint8 [num_pages, 64, 656] */
    const int32_t* block_table;  /* int32 [B, max_pages] */
    const int32_t* insert_pos;   /* int32 [B] */
    int32_t        max_pages;
    int32_t        reserved0;
    int64_t        num_pages;
    int32_t*       status;       /* optional int32[4], zeroed by the caller */
} Dsv4CacheDest;

/*
 * HCA compressor (cache-write side of the dense path): every block of m rows
 * becomes one row; per channel, softmax over the m gating logits Z + bias weights
 * the m value rows C.  Follows the reduce of the reference's compressor_simple
 * (bench/bench/reference.py:108-122) and replaces the reference's kernel stub
 * hca_compress (hca/sm100/kernel.cu:34-78, which writes FP8 with a scale of one).
 * Output, either or both:
 *   out  - dense BF16 [B, n/m, c];
 *   dst  - (c must be 576) the BF16-rounded row quantised with the cache's recipe
 *          (FP32 absmax/448 scale per 128 latent elements, e4m3 round-to-nearest-even
 *          saturating, RoPE tail kept in BF16: the reference quantiser
 *          bench/bench/decode.py:92-114 with this cache's tile and scale type) and
 *          written as entry insert_pos[b] + i of request b.  Bit-identical to calling
 *          dsv4_kv_quantize_insert on `out`.
 * Requires c % 8 == 0, strides % 8 == 0 and 16-byte aligned pointers
 * (cudaErrorInvalidValue otherwise).  Any m >= 1 with n % m == 0.
 */
typedef struct Dsv4HcaCompressParams {
    int32_t B;              /* batch */
    int32_t n;              /* rows per request, divisible by m */
    int32_t c;              /* channels */
    int32_t m;              /* compression rate (128 in the model) */
    const void* C;          /* bf16 [B, n, c] value stream */
    const void* Z;          /* bf16 [B, n, c] gating logits */
    const void* bias;       /* bf16 [m, c] */
    int64_t stride_b;       /* element strides of C and Z */
    int64_t stride_n;
    void*   out;            /* bf16 [B, n/m, c] contiguous, or NULL */
    const Dsv4CacheDest* dst;   /* or NULL */
} Dsv4HcaCompressParams;

int dsv4_hca_compress_fwd(const Dsv4HcaCompressParams* p, void* stream);

/*
 * Quantise BF16 rows [B, T, 576] (512 latent + 64 RoPE) into cache entries and
 * write them at logical positions insert_pos[b] .. insert_pos[b] + T - 1 (or
 * n_rows[b] rows when n_rows is given).  The step that follows the CSA compressor
 * (dsv4_csa_compress_reduce_fwd) or any other producer of new cache rows.  The
 * quantiser is the reference's recipe (bench/bench/decode.py:92-114) with this
 * cache's FP32 scale per 128 elements; results are bit-identical to the CPU
 * restatement.
 */
typedef struct Dsv4KvQuantizeInsertParams {
    int32_t B;
    int32_t T;
    const void* rows;       /* bf16 [B, T, 576] */
    int64_t stride_b;       /* element strides, multiples of 8 */
    int64_t stride_t;
    const int32_t* n_rows;  /* optional int32 [B] */
    const Dsv4CacheDest* dst;
} Dsv4KvQuantizeInsertParams;

int dsv4_kv_quantize_insert(const Dsv4KvQuantizeInsertParams* p, void* stream);

/*
 * Plain-SIMT validation kernels: the same three operations computed without
 * tensor cores, one head per thread block.  They exist so that large cases can
 * be cross-checked on the device; they are slow and are not the product path.
 * No counterpart in the reference.
 */
int dsv4_csa_sparse_decode_simt(const Dsv4CsaSparseDecodeParams* p, void* stream);
int dsv4_hca_dense_decode_simt(const Dsv4HcaDenseDecodeParams* p, void* stream);

/* Test switches, process-wide (read once per call); 0 = product behaviour.  bit6: launch the split-KV
 * merge and the indexer's top-k as ordinary kernels instead of as programmatic dependents of the kernel
 * before them.  No counterpart in the reference. */
void dsv4_debug_set_flags(int flags);

/* Test aid for the error path of the bounded waits.  wait_ns: limit of every wait inside the decode
 * kernels and the indexer's scoring kernel (0 = the default, 2 s).  drop_tile >= 0: in every decode
 * block the loaders withhold the hand-over of the tile with that running number (in every block of the
 * scoring kernel the MMA warp withholds the "accumulator full" signal of that tile), so that the waits
 * behind it run out; the kernel must then return with `status` naming the wait (no trap, no fault) and
 * the next launch must be unaffected.  drop_tile = -1 switches it off.  The reference's counterpart is the trap after a
 * cycle budget in hca/sm100/helpers.h:183-206. */
void dsv4_debug_set_wait(unsigned long long wait_ns, int drop_tile);

/* Library identification: (major << 16) | minor. */
int dsv4_attn_version(void);

#ifdef __cplusplus
}
#endif

#endif /* DSV4_ATTN_H_ */
