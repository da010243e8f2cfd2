/* Shared between the C host (clef_cuda_omni.c) and the CUDA translation units.
 * Plain C declarations only: launchers take raw pointers and a cudaStream_t. */
#ifndef OMNI_INTERNAL_H
#define OMNI_INTERNAL_H

#include <stdint.h>
#include <cuda.h>
#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    OMNI_H = 2048, OMNI_F = 768, OMNI_E = 128, OMNI_TOP = 8,
    OMNI_NH = 32, OMNI_NKV = 4, OMNI_HD = 128, OMNI_QKV = (OMNI_NH + 2 * OMNI_NKV) * OMNI_HD,   /* attention half: 32 query, 4 key/value heads of 128 */
    OMNI_CHUNK = 16384,                    /* tokens per arena pass */
    OMNI_ROWS = OMNI_CHUNK * OMNI_TOP,     /* permuted rows per pass */
    OMNI_SEG = 256,                        /* assignments per sort segment (one warp) */
    OMNI_MAX_SEGS = OMNI_ROWS / OMNI_SEG,
    OMNI_TILE_N = 256,                     /* token rows per expert-GEMM tile */
    OMNI_MAX_TTILES = OMNI_ROWS / OMNI_TILE_N + OMNI_E,
};

/* status word bits (clef_omni_complete) */
enum { OMNI_ST_NONFINITE = 1u, OMNI_ST_BAD_ID = 8u, OMNI_ST_TIMEOUT = 16u, OMNI_ST_EP_OVERFLOW = 32u,
       /* which bounded wait ran out (set together with OMNI_ST_TIMEOUT) */
       OMNI_ST_TIMEOUT_BARRIER = 64u, OMNI_ST_TIMEOUT_ARRIVAL = 128u,
       /* the exact pass found a tensor-core logit further from its exact value than the bound the
        * near-tie test assumes: rows that were not re-decided may carry a wrong order */
       OMNI_ST_ROUTER_EPS = 256u,
       /* nonfinite values met while preparing q, k, v (the reference's attention status bit, clef.metal:2120) */
       OMNI_ST_ATTN_NONFINITE = 2u };

/* Bound assumed on |tensor-core logit - exact logit| for one row: `eps` for rows whose largest
 * |logit| is at most OMNI_EPS_REF_SCALE, growing in proportion beyond that (the FP32 accumulation
 * error of a 2048-term sum scales with the magnitude of its partial sums). */
#define OMNI_EPS_REF_SCALE 4.0f
#ifdef __CUDACC__
__host__ __device__
#endif
static inline float omni_row_eps(float eps, float max_abs_logit) {
    const float s = max_abs_logit * (1.0f / OMNI_EPS_REF_SCALE);
    return s > 1.0f ? eps * s : eps;
}

/* One token tile of one expert: rows [row0, row0+len) of the permuted buffers. */
/* group = index of the expert's first tile | (its tile count << 16) */
typedef struct { int32_t expert, row0, len, group; } omni_ttile;

/* Device-resident sort/tile state produced by the assignment kernels. */
typedef struct {
    int32_t *counts;       /* [E]                                     */
    int32_t *offsets;      /* [E+1] exclusive prefix sum of counts    */
    int32_t *rowmap;       /* [rows*8] token of each permuted row     */
    int32_t *slots;        /* [rows*8] permuted row of assignment i   */
    int32_t *segcount;     /* [MAX_SEGS][E] per-segment histograms, then exclusive bases */
    omni_ttile *ttiles;    /* [MAX_TTILES] expert-major, an expert's rows in near-equal tiles */
    int32_t *n_ttiles;     /* [1]                                     */
    int32_t *sched;        /* [8] work counters: [0] gate/up, [1..] down (one per launch group), zeroed by the scan */
    uint32_t *status;      /* [1]                                     */
    int32_t *n_flag;       /* [2] rows flagged for the exact pass: the scan moves [0] to [1] and clears [0] for the next pass */
    int32_t *done;         /* [128] epilogue warps of the gate/up kernel that have stored their part of an expert's rows; zeroed by the scan (may be NULL) */
    int32_t *done_need;    /* [128] what done[e] reaches when expert e's rows are complete: 8 warps x 6 weight tiles x token tiles */
    int32_t longest_first; /* tile list in order of falling tile length (else in expert order) */
    omni_ttile *ttiles_down; /* the same tiles in expert order, for the down kernel (may be NULL: it then reads ttiles) */
} omni_sort_state;

/* Expert parallelism: every rank's view of every rank's exchange buffers (index = rank). */
enum { OMNI_EP_MAX = 8, OMNI_EP_BUFFERS = 6, OMNI_EP_GROUPS = 4, OMNI_EP_BUCKETS = OMNI_EP_MAX * OMNI_EP_GROUPS,
       OMNI_EP_COUNT_STRIDE = OMNI_E + OMNI_EP_BUCKETS };   /* ints one rank publishes: expert counts, then bucket counts */
typedef struct {
    int32_t rank, world;
    void *xg[OMNI_EP_MAX];          /* [ROWS][2048] bf16: token rows received, expert-major      */
    void *dret[OMNI_EP_MAX];        /* [ROWS][2048] bf16: expert outputs returned, source order  */
    int32_t *rowinfo[OMNI_EP_MAX];  /* [ROWS] (source rank << 20) | source permuted row          */
    int32_t *counts[OMNI_EP_MAX];   /* [EP_MAX][COUNT_STRIDE] per-expert and per-bucket counts of every rank */
    int32_t *grow[OMNI_EP_MAX];     /* [ROWS] received row (index into xg) that holds each expert-major row's token */
    uint32_t *flags[OMNI_EP_MAX];   /* [EP_MAX] barrier epochs, written by the peers; from word
                                       OMNI_EP_READY_WORD on: rows arrived per local expert       */
} omni_ep_peers;
/* flag words: [0, EP_MAX) barrier epochs; [SYNC_WORD, +EP_MAX) sync counts, then EP_MAX epochs
 * published for realignment; from READY_WORD on, rows arrived per local expert group */
enum { OMNI_EP_SYNC_WORD = 16, OMNI_EP_READY_WORD = 64, OMNI_EP_FLAG_WORDS = 64 + 128 };
/* local experts are announced as "arrived" in groups of this many (four groups per rank) */
#ifdef __CUDACC__
__host__ __device__
#endif
static inline int omni_ep_group_size(int world) { const int el = OMNI_E / world; return el >= OMNI_EP_GROUPS ? el / OMNI_EP_GROUPS : 1; }

/* What the sender side of the de-duplicated dispatch works from (all device pointers of this rank).
 * A token goes ONCE to every rank that owns at least one of its experts, into the bucket
 * (owner, first group of that owner's experts that needs it). */
typedef struct {
    const int32_t *tok_slot;      /* [T][EP_MAX]  (group << 24) | position of the token in its bucket for that owner, -1: not sent there */
    const int32_t *bucket_list;   /* [BUCKETS][CHUNK] tokens of each bucket */
    const int32_t *send_cnt;      /* [BUCKETS] tokens this rank sends per bucket */
    const int32_t *recv_base;     /* [BUCKETS] first row of this rank's tokens of a bucket in the owner's receive buffer */
    const int32_t *send_base;     /* [128] first expert-major row of this rank's rows of an expert on its owner */
    const int32_t *rowmap, *offsets;
    const void *xn;               /* [T][2048] bf16 */
} omni_ep_send;

/* ---- plain kernels (omni_kernels.cu) ---- */
cudaError_t omni_launch_router_simple(const void *xn, const void *router, const float *bias, int T,
                                      float *logits, cudaStream_t s);
cudaError_t omni_launch_select(const float *logits, int T, float eps, int exact_all, int32_t *ids, float *weights,
                               int32_t *flag_rows, int32_t *n_flag, uint32_t *status, cudaStream_t s);
/* logits: the approximate values on entry; on return every logit the exact pass evaluated holds
 * (float)exact, and low (may be NULL) the remainder (float)(exact - hi) */
cudaError_t omni_launch_recheck(int32_t *segcount, const void *xn, const void *router, const float *bias, float *logits,
                                float *low, const int32_t *flag_rows, const int32_t *n_flag, int T, float eps,
                                int32_t *ids, float *weights, uint32_t *status, cudaStream_t s);
cudaError_t omni_launch_router_exact(const void *xn, const void *router, const float *bias, int T,
                                     double *logits, cudaStream_t s);
cudaError_t omni_launch_route_pairs(const float *hi, const float *lo, int rows, int32_t *ids, float *weights,
                                    uint32_t *status, cudaStream_t s);
/* have_counts: st.segcount already holds the per-segment expert counts of ids (the router kernel wrote them) */
cudaError_t omni_launch_assign(const int32_t *ids, int rows, omni_sort_state st, int have_counts, cudaStream_t s);
/* xn[rows][2048] BF16 = RMSNorm of x[rows][2048] FP32 with FP32 weights w[2048] */
cudaError_t omni_launch_rmsnorm(const float *x, const float *w, float eps, int rows, void *xn, cudaStream_t s);
cudaError_t omni_launch_gather(const void *xn, const int32_t *rowmap, int rows8, void *xg, cudaStream_t s);
cudaError_t omni_launch_combine(const void *d, const int32_t *ids, const float *weights, const int32_t *slots,
                                float *x, int T, cudaStream_t s);
cudaError_t omni_launch_gateup_simple(const void *xg, const void *gate_up, const int32_t *offsets, int rows8, void *h,
                                      cudaStream_t s);
cudaError_t omni_launch_down_simple(const void *h, const void *down, const int32_t *offsets, int rows8, void *d,
                                    cudaStream_t s);
cudaError_t omni_launch_fill_u32(void *p, uint32_t v, size_t words, cudaStream_t s);
cudaError_t omni_launch_touch(const void *p, uint32_t *sink, cudaStream_t s);
cudaError_t omni_launch_trace(const float *logits, const float *low, const int32_t *ids, const float *weights, int rows, int start,
                              int first, int captured, int layer, void *trace, cudaStream_t s);

/* the sort with its scratch in a static device array (no allocation); *max_rows = its limit */
cudaError_t omni_noalloc_assign(const int32_t *ids, int rows, int32_t *counts, int32_t *offsets, int32_t *rowmap,
                                int32_t *slots, uint32_t *status, cudaStream_t s, int *max_rows);

/* ---- tcgen05 kernels (omni_sm100.cu) ---- */
cudaError_t omni_sm100_configure(void);   /* opt-in shared-memory sizes; call once per device */
/* ---- router (omni_router.cu) ---- */
cudaError_t omni_router_configure(void);
int omni_router_tile(int T, int n_sm);     /* tokens per CTA: 32 while that gives at most one CTA per SM, else 128 */
/* tm_x: the activations with a box of 64 K elements x nt rows (nt = omni_router_tile(T, n_sm)) */
cudaError_t omni_launch_router_sm100(const CUtensorMap *tm_x, int nt, const CUtensorMap *tm_w, const float *bias, int T,
                                     float eps, int exact_all, float *logits, int32_t *ids, float *weights,
                                     int32_t *flag_rows, int32_t *n_flag, uint32_t *status, unsigned long long *dbg,
                                     int32_t *segcount, cudaStream_t s);
/* segcount (may be NULL): the kernel also writes the per-segment expert counts of the counting
 * sort for the ids it selected; omni_launch_recheck must then be given the same pointer so that
 * the rows it re-decides move their counts */
/* tm_x4 / tm_h4: four maps of the same buffer with box heights 32, 64, 128 and 256 rows */
/* ready/need (may be NULL): rows that have arrived / must arrive per expert before its token
 * rows may be read (expert parallelism: the rows are written by other GPUs while this runs).
 * gather_src/gather_rows (may be NULL): the kernel fetches token row i of the permuted order from
 * row gather_rows[i] of gather_src ([rows][2048] BF16) itself and tm_x4 is not used */
cudaError_t omni_launch_gateup_sm100(const CUtensorMap *tm_w, const CUtensorMap *tm_x4, const omni_sort_state st,
                                     void *h, const uint32_t *ready, const int32_t *need, int group_size,
                                     const void *gather_src, const int32_t *gather_rows, int early_dependents, int announce,
                                     int n_sm, cudaStream_t s);
/* tile_bounds (may be NULL) + group: restrict the launch to tiles [tile_bounds[group], tile_bounds[group+1]).
 * early_dependents (both launchers): let blocks of the next kernel in the stream become resident
 * while this one runs; pass 0 when the grid leaves SMs free for kernels of another stream */
/* announce (gate/up) + chained (down): the gate/up kernel counts, per expert, the epilogue warps
 * that have stored their rows (st.done); the down kernel launched behind it then does not wait for
 * the whole gate/up grid but, per expert, for st.done[e] to reach st.done_need[e], so its blocks
 * start on the SMs the first gate/up blocks leave while the last ones are still working. */
cudaError_t omni_launch_down_sm100(const CUtensorMap *tm_w, const CUtensorMap *tm_h4, const omni_sort_state st,
                                   void *d, const int32_t *tile_bounds, int group, int early_dependents, int chained,
                                   int n_sm, cudaStream_t s);

/* ---- expert products on pairs of SMs (omni_expert.cu) ---- */
cudaError_t omni_expert_configure(void);  /* opt-in shared-memory sizes; call once per device */
/* ctas: 2 = clusters of two CTAs driving tcgen05.mma.cta_group::2, 1 = the same code on single CTAs.
 * tm_w3: three-dimensional map of the gate/up matrix {K, gate|up, row} with box {64, 2, 64}: gate
 * and up rows of the same intermediate column arrive interleaved.  Other arguments as in
 * omni_launch_gateup_sm100. */
cudaError_t omni_launch_gateup_pair(int ctas, const CUtensorMap *tm_w3, const CUtensorMap *tm_x4, const omni_sort_state st,
                                    void *h, const uint32_t *ready, const int32_t *need, int group_size,
                                    const void *gather_src, const int32_t *gather_rows, const omni_ep_peers *dispatch_to,
                                    const omni_ep_send *send, int early_dependents, int n_sm, cudaStream_t s);
/* dispatch_to/send (may be NULL): expert parallelism -- four more warps per CTA send this rank's
 * token rows, each once per owner rank, into the owners' receive buffers (gather_src of the
 * owner) with the row map (gather_rows of the owner) and the origin tags, and count themselves on
 * the owners' arrival counters, which `ready` of every rank waits for, group by group.
 * return_to/rowinfo (may be NULL): result row i is written to row (rowinfo[i] & 0xfffff) of
 * return_to->dret[rowinfo[i] >> 20] (the rank the token came from) instead of row i of d */
cudaError_t omni_launch_down_pair(int ctas, const CUtensorMap *tm_w, const CUtensorMap *tm_h4, const omni_sort_state st,
                                  void *d, const omni_ep_peers *return_to, const int32_t *rowinfo, int early_dependents, int n_sm,
                                  cudaStream_t s);

/* ---- attention half (omni_attn.cu; the two projections run on the kernel of omni_expert.cu) ---- */
cudaError_t omni_attn_configure(void);
/* tile list that cuts T token rows into tiles of one "expert"; counters[0..1] are cleared (work counters of the two projections) */
cudaError_t omni_launch_dense_tiles(int T, omni_ttile *ttiles, int32_t *n_ttiles, int32_t *counters, cudaStream_t s);
/* which: 0 = q|k|v projection (out_bf16 [T][5120]), 1 = output projection (added into resid [T][2048]) */
cudaError_t omni_launch_dense_pair(int which, const CUtensorMap *tm_w, const CUtensorMap *tm_tok4, const omni_sort_state st,
                                   int32_t *work_counter, void *out_bf16, float *resid, int n_sm, cudaStream_t s);
/* qkv [T][5120] BF16 -> Q [32][T][128], K [4][T][128], Vt [4][128][vpitch] (column vcol[t] for token t), BF16;
 * pos [T][3] positions (temporal, row, column); head_stride: rows between two heads of Q and K */
cudaError_t omni_launch_attn_prep(const void *qkv, const float *qw, const float *kw, const int32_t *pos, const int32_t *vcol, int T,
                                  int head_stride, int vpitch, float eps, double theta, void *Q, void *K, void *Vt, uint32_t *status,
                                  cudaStream_t s);
/* tiles: [n_tiles] x {record start, first query row, rows (<= 128), Vt column of the record start}; out [T][4096] BF16 */
cudaError_t omni_launch_attention(const CUtensorMap *tm_q, const CUtensorMap *tm_k, const CUtensorMap *tm_vt, const void *tiles,
                                  int n_tiles, int T, void *out, uint32_t *status, cudaStream_t s);

/* Programmatic dependent launch of the pass's kernel chain (process-wide, default on) */
void omni_set_dependent_launch(int on);
int omni_dependent_launch_enabled(void);

/* ---- expert parallel (omni_ep.cu) ---- */
/* limit_ns = 0 (here and below): the default bound of 2 s on the wait for the other ranks */
cudaError_t omni_launch_ep_plan(const omni_ep_peers *pe, uint32_t epoch, omni_sort_state st, int32_t *send_base,
                                int32_t *n_local_rows, int32_t *need, int32_t *bucket_cnt, int32_t *send_cnt, int32_t *recv_base,
                                uint64_t limit_ns, cudaStream_t s);
/* tokens of this rank -> buckets (owner, first group that needs the token); bucket_cnt must be zero on entry
 * (the plan kernel leaves it so) */
cudaError_t omni_launch_ep_buckets(const int32_t *ids, int T, int world, int32_t *tok_slot, int32_t *bucket_cnt,
                                   int32_t *bucket_list, cudaStream_t s);
/* realignment barrier: result[0] = agreed sync count, result[1] = agreed epoch (written on success only) */
cudaError_t omni_launch_ep_sync(const omni_ep_peers *pe, uint32_t count, uint32_t epoch, uint32_t *status, uint32_t *result,
                                uint64_t limit_ns, cudaStream_t s);
cudaError_t omni_launch_ep_barrier(const omni_ep_peers *pe, uint32_t epoch, uint32_t *status, uint64_t limit_ns,
                                   cudaStream_t s);
cudaError_t omni_launch_ep_dispatch(const omni_ep_peers *pe, const void *xn, const int32_t *rowmap, const int32_t *offsets,
                                    const int32_t *send_base, int rows8, int signal, int n_sm, cudaStream_t s);
#ifdef __cplusplus
}
#endif
#endif
