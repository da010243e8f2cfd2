// The two grouped expert products of the Clef-Omni MoE block on single CTAs (sm_100a, tcgen05
// cta_group::1): the schedule used on one GPU.  omni_expert.cu holds the CTA-pair schedule that
// also moves the rows of expert parallelism; omni_router.cu the router.
//   * expert_gemm_kernel<GATEUP>  per expert: h = silu(Xe Wg^T) * (Xe Wu^T), SwiGLU in the epilogue
//                           (reference: metal/clef.metal:2455-2492, omni_expert_gemm + omni_swiglu);
//                           the kernel also fetches the expert's token rows through
//                           the permutation itself (metal/clef.metal:2445-2453, omni_gather)
//   * expert_gemm_kernel<DOWN>    per expert: d = He Wd^T            (clef.metal:2455-2482)
//
// Orientation of the expert products: the WEIGHT rows are the MMA M dimension (always a full
// 128), the expert's TOKEN rows are the N dimension (16..256 in steps of 16).  A ragged expert
// therefore costs its real row count rounded up to 16, not to a 128-row tile, and every
// weight tile is streamed from HBM by exactly one CTA when the expert has <= 256 rows.
//
// Operands reach shared memory through per-CTA TMA loads (cp.async.bulk.tensor, 128-byte
// swizzle), the gathered token rows through 16-byte cp.async into the same swizzled layout; no
// cluster multicast is used anywhere.  Every wait on an mbarrier is bounded: when
// it runs out the CTA raises OMNI_ST_TIMEOUT in the status word, drains what it issued, frees
// its TMEM and returns.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "omni_internal.h"
#include "omni_pdl.cuh"
#include "omni_ptx.cuh"

namespace {

// ====================================================================== grouped expert products
enum { MODE_GATEUP = 0, MODE_DOWN = 1 };

// Weights come from HBM (about 2 us away under load), token rows mostly from L2: the two operands
// therefore have their own shared-memory rings, the weight ring deeper than the token ring,
// each filled by its own producer thread so the weight loads can run further ahead.
template <int MODE> struct GemmCfg;
template <> struct GemmCfg<MODE_GATEUP> {
    static constexpr int KTOT = OMNI_H, NACC = 2, NBUF = 1, W_STAGES = 4, T_STAGES = 3, MTILES = OMNI_F / 128;
    static constexpr int W_ROWS_PER_EXPERT = 2 * OMNI_F, OUT_COLS = OMNI_F;
};
template <> struct GemmCfg<MODE_DOWN> {
    static constexpr int KTOT = OMNI_F, NACC = 1, NBUF = 2, W_STAGES = 6, T_STAGES = 4, MTILES = OMNI_H / 128;
    static constexpr int W_ROWS_PER_EXPERT = OMNI_H, OUT_COLS = OMNI_H;
};

constexpr int GEMM_THREADS = 384;            // warp 0 scheduler + weight TMA, 1 MMA, 2 TMEM, 3 token TMA, 4..11 epilogue
constexpr int EPI_WARPS = 8;
constexpr int GATHER_THREADS = 64;                  // warps 2 and 3 when the kernel gathers its token rows itself
constexpr int T_TILE_BYTES = OMNI_TILE_N * BK * 2;   // 32 KiB: up to 256 token rows

template <int MODE> struct GemmSmem {
    static constexpr int W_BYTES = GemmCfg<MODE>::NACC * A_TILE_BYTES;
    static constexpr int RING_BYTES = GemmCfg<MODE>::W_STAGES * W_BYTES + GemmCfg<MODE>::T_STAGES * T_TILE_BYTES;
    static constexpr int TOTAL_BYTES = RING_BYTES + 1024 + 512;
};
static_assert(GemmSmem<MODE_GATEUP>::TOTAL_BYTES <= 232448 && GemmSmem<MODE_DOWN>::TOTAL_BYTES <= 232448, "shared memory budget");

// silu(g) * u with silu(g) = g * sigmoid(g) = (g/2) * (1 + tanh(g/2)): one special-function
// instruction per element instead of two (exp and reciprocal).  The epilogue holds tensor memory
// while it computes this and is bound by the special-function unit (one warp instruction per 8
// cycles), so the count of such instructions is what matters.  tanh.approx.f32 is accurate to
// about 2^-11 absolute; the result is rounded to BF16 (2^-9 relative) right after.
__device__ __forceinline__ float silu_mul(float g, float u) {
    const float hg = 0.5f * g;
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(hg));
    return fmaf(hg, t, hg) * u;
}

// Work distribution.  The work list is expert-major: for one expert, every (weight tile m,
// token tile j) pair is consecutive, so CTAs that run at the same time share either the token
// rows or the weight rows through L2 and each weight byte leaves HBM once even when an expert
// has more than one token tile.  Items differ in cost, so CTAs claim them one at a time from a
// device counter; warp 0 claims and hands the decoded item to the token producer, the MMA
// thread and the epilogue warps through a small shared-memory ring.
struct WorkSlot { int expert, row0, len, m; };
constexpr int RING = 4;

template <int MODE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
expert_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ TokMaps tm_tok,
                   const omni_ttile *__restrict__ ttiles, const int32_t *__restrict__ n_ttiles,
                   int32_t *__restrict__ work_counter, __nv_bfloat16 *__restrict__ out, uint32_t *__restrict__ status,
                   const uint32_t *__restrict__ ready, const int32_t *__restrict__ need, int group_size,
                   const int32_t *__restrict__ tile_bounds, int tile_group,
                   const __nv_bfloat16 *__restrict__ gather_src, const int32_t *__restrict__ gather_rows,
                   int early_dependents, int32_t *__restrict__ done, int chained) {
    using C = GemmCfg<MODE>;
    constexpr int KSTAGES = C::KTOT / BK;
    constexpr int WS = C::W_STAGES, TS = C::T_STAGES;
    constexpr int W_BYTES = GemmSmem<MODE>::W_BYTES;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t tok_base = smem_base + WS * W_BYTES;
    const uint32_t bar_base = smem_base + GemmSmem<MODE>::RING_BYTES;   // 8-byte aligned
    // barriers: wfull[WS] wempty[WS] tfull[TS] tempty[TS] acc_full[2] acc_empty[2] drain item_full[RING] item_empty[RING]
    auto wfull_bar = [&](int s) { return bar_base + 8u * s; };
    auto wempty_bar = [&](int s) { return bar_base + 8u * (WS + s); };
    auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * WS + s); };
    auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * WS + TS + s); };
    auto afull_bar = [&](int b) { return bar_base + 8u * (2 * WS + 2 * TS + b); };
    auto aempty_bar = [&](int b) { return bar_base + 8u * (2 * WS + 2 * TS + 2 + b); };
    const uint32_t drain_bar = bar_base + 8u * (2 * WS + 2 * TS + 4);
    auto ifull_bar = [&](int r) { return bar_base + 8u * (2 * WS + 2 * TS + 5 + r); };
    auto iempty_bar = [&](int r) { return bar_base + 8u * (2 * WS + 2 * TS + 5 + RING + r); };
    constexpr int N_BARS = 2 * WS + 2 * TS + 5 + 2 * RING;
    static_assert(N_BARS * 8 + 16 + 8 * 4 + 8 * 4 + RING * 16 <= 512, "barrier block");
    uint8_t *misc = smem_raw + (bar_base - smem_u32(smem_raw)) + 8 * N_BARS;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(misc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(misc + 4);
    volatile int *armed_w = reinterpret_cast<volatile int *>(misc + 16);        // [8] parity armed per weight stage, -1 none
    volatile int *armed_t = reinterpret_cast<volatile int *>(misc + 16 + 32);   // [8] same for the token ring
    volatile WorkSlot *ring = reinterpret_cast<volatile WorkSlot *>(misc + 16 + 64);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < WS; s++) { mbar_init(wfull_bar(s), 1); mbar_init(wempty_bar(s), 1); }
        for (int s = 0; s < TS; s++) { mbar_init(tfull_bar(s), gather_src ? GATHER_THREADS : 1); mbar_init(tempty_bar(s), 1); }
        for (int s = 0; s < 8; s++) { armed_w[s] = -1; armed_t[s] = -1; }
        for (int b = 0; b < 2; b++) { mbar_init(afull_bar(b), 1); mbar_init(aempty_bar(b), EPI_WARPS); }
        mbar_init(drain_bar, 1);
        for (int r = 0; r < RING; r++) { mbar_init(ifull_bar(r), 1); mbar_init(iempty_bar(r), (gather_src ? GATHER_THREADS : 1) + 1 + EPI_WARPS); }
        *abort_flag = 0;
        fence_mbar_init();
        prefetch_tmap(&tm_w);
        for (int i = 0; i < 4; i++) prefetch_tmap(&tm_tok.m[i]);
    }
    if (warp == 2) { tmem_alloc(smem_u32((const void *)tmem_slot), 512); tmem_relinquish(); }
    // Chained behind the gate/up kernel, the down kernel does not wait for that whole grid: what it
    // reads of it (rows of h) it takes expert by expert once `ready` says they are complete.  The
    // kernels before gate/up had completed before gate/up let this grid start; their results (the
    // tile list) are read past L1 below.
    if (!chained) dep_wait();   // everything above overlaps the tail of the previous kernel
    // Blocks of the next kernel that become resident early sit on whatever SM is free.  When
    // this grid leaves SMs free on purpose (for copy kernels of another stream), it must not
    // invite them.
    if (early_dependents) dep_launch();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // the launch covers work items [work_lo, n_work): everything, or one group of experts
    const int work_lo = tile_bounds ? tile_bounds[tile_group] * C::MTILES : 0;
    const int n_tt = __ldcg(n_ttiles);
    const int n_work = tile_bounds ? min(tile_bounds[tile_group + 1], n_tt) * C::MTILES : n_tt * C::MTILES;

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------- scheduler + weight producer
        // Claiming and decoding an item costs an atomic and two dependent global loads (~2 us).
        // They are software-pipelined behind the TMA issue loop: while item i is being loaded,
        // item i+1 is decoded (its claim came back one iteration ago) and item i+2 is claimed.
        PipeState p, wr;
        const uint64_t pol_w1 = l2_policy_evict_first(), pol_keep = l2_policy_evict_last();
        auto tile_at = [&](int i) {                           // past L1: a chained launch starts before its predecessor ends
            const int4 v = __ldcg(reinterpret_cast<const int4 *>(ttiles) + i);
            return omni_ttile{v.x, v.y, v.z, v.w};
        };
        auto lookup = [&](int w, int &m, int &cnt) {          // item -> (weight tile m, tile-list index)
            const omni_ttile t0 = tile_at(w / C::MTILES);
            const int first = t0.group & 0xffff;
            cnt = t0.group >> 16;
            const int local = w - first * C::MTILES;
            m = local / cnt;
            return first + local % cnt;
        };
        int cur_m = 0, cur_cnt = 1;
        omni_ttile cur = omni_ttile{0, 0, -1, 0};
        int w0 = work_lo + atomicAdd(work_counter, 1);
        int w1 = work_lo + atomicAdd(work_counter, 1);        // index of the item after the current one
        if (w0 < n_work) cur = tile_at(lookup(w0, cur_m, cur_cnt));
        for (;;) {
            if (!mbar_wait(iempty_bar(wr.stage), wr.phase ^ 1u, abort_flag, status)) break;
            if (cur.len < 0) {
                ring[wr.stage].len = -1;                      // tells the consumers to stop
                mbar_arrive(ifull_bar(wr.stage));
                break;
            }
            ring[wr.stage].expert = cur.expert; ring[wr.stage].row0 = cur.row0;
            ring[wr.stage].len = cur.len; ring[wr.stage].m = cur_m;
            mbar_arrive(ifull_bar(wr.stage));
            wr.advance(RING);
            const int w2 = work_lo + atomicAdd(work_counter, 1);   // consumed two iterations from now
            const bool has_next = w1 < n_work;
            omni_ttile head = omni_ttile{0, 0, 0, 0};
            if (has_next) head = tile_at(w1 / C::MTILES);      // first dependent load: in flight during the loop below
            int nxt_m = 0, nxt_cnt = 1;
            const int wrow = cur.expert * C::W_ROWS_PER_EXPERT + cur_m * 128;
            // a weight tile is read once per token tile of its expert: keep it in L2 while
            // the expert's other token tiles (claimed by neighbouring CTAs) still need it
            const uint64_t pol_w = cur_cnt > 1 ? pol_keep : pol_w1;
            omni_ttile nxt = omni_ttile{0, 0, -1, 0};
            bool ok = true;
            for (int ks = 0; ks < KSTAGES; ks++) {
                if (ks == KSTAGES / 4 && has_next) {           // first load has landed: issue the second
                    const int first = head.group & 0xffff;
                    nxt_cnt = head.group >> 16;
                    const int local = w1 - first * C::MTILES;
                    nxt_m = local / nxt_cnt;
                    nxt = tile_at(first + local % nxt_cnt);
                }
                ok = mbar_wait(wempty_bar(p.stage), p.phase ^ 1u, abort_flag, status);
                if (!ok) break;
                const uint32_t sa = smem_base + p.stage * W_BYTES;
                armed_w[p.stage] = (int)p.phase;
                mbar_expect_tx(wfull_bar(p.stage), W_BYTES);
                tma_load_2d_hint(sa, &tm_w, ks * BK, wrow, wfull_bar(p.stage), pol_w);
                if (C::NACC == 2) tma_load_2d_hint(sa + A_TILE_BYTES, &tm_w, ks * BK, wrow + OMNI_F, wfull_bar(p.stage), pol_w);
                p.advance(WS);
            }
            if (!ok) break;
            cur = nxt; cur_m = nxt_m; cur_cnt = nxt_cnt;
            w1 = w2;
        }
    } else if ((warp == 2 || warp == 3) && gather_src) {
        // ---------------------------------------------------------- token producer, gathering
        // The token rows of an expert are scattered over the activation matrix.  Instead of a
        // kernel that first copies them into expert order (a write and a read of T*8 rows in
        // HBM), these 64 threads fetch them here: 16-byte asynchronous copies, eight threads per
        // 128-byte row segment, stored in the 128-byte-swizzled layout the MMA descriptors
        // expect (chunk c of row r at c ^ (r & 7) inside its 8-row group).  A stage is handed to
        // the MMA thread two stages after it was issued, once this thread's copies have landed
        // and are ordered before the tensor core's reads.
        constexpr int LAG = 2;
        static_assert(TS > LAG, "token ring too short for the copy lag");
        const uint64_t pol_t = l2_policy_evict_last();    // every row is read again for each weight tile
        const int gt = threadIdx.x - 64;                  // 0..63
        const int c = gt & 7, rb = gt >> 3;               // chunk of the row segment, row inside the 8-row group
        const uint32_t dst_off = (uint32_t)(rb * 128 + ((c ^ rb) << 4));
        const char *src0 = reinterpret_cast<const char *>(gather_src) + c * 16;
        PipeState p, pend, wr;
        int off[OMNI_TILE_N / 8], off_next[OMNI_TILE_N / 8];   // byte offsets of this thread's rows, -1 past the tile
        // takes the next item from the ring and starts the loads of its row indices
        auto next_item = [&](int (&o)[OMNI_TILE_N / 8]) -> int {
            if (!mbar_wait(ifull_bar(wr.stage), wr.phase, abort_flag, status)) return -1;
            const int row0 = ring[wr.stage].row0, len = ring[wr.stage].len;
            mbar_arrive(iempty_bar(wr.stage));
            wr.advance(RING);
#pragma unroll
            for (int i = 0; i < OMNI_TILE_N / 8; i++) {
                const int r = rb + 8 * i;
                o[i] = r < len ? gather_rows[row0 + r] * (OMNI_H * 2) : -1;
            }
            return len;
        };
        int len = next_item(off);
        while (len >= 0) {
            bool ok = true;
            for (int ks = 0; ks < KSTAGES; ks++) {
                if (ks >= LAG) {
                    // hand over the oldest stage before blocking on a free one: the MMA thread
                    // must never wait for this loop to issue further copies
                    cp_async_wait<LAG - 1>();
                    fence_proxy_async_smem();
                    mbar_arrive(tfull_bar(pend.stage));
                    pend.advance(TS);
                }
                ok = mbar_wait(tempty_bar(p.stage), p.phase ^ 1u, abort_flag, status);
                if (!ok) break;
                const uint32_t sb = tok_base + p.stage * T_TILE_BYTES + dst_off;
                const char *src = src0 + ks * (BK * 2);
#pragma unroll
                for (int i = 0; i < OMNI_TILE_N / 8; i++)
                    if (off[i] >= 0) cp_async16(sb + i * 1024, src + off[i], pol_t);
                cp_async_commit();
                p.advance(TS);
            }
            if (!ok) break;
            // the next item's row indices travel while the last two stages of this one land
            len = next_item(off_next);
            cp_async_wait<1>();
            fence_proxy_async_smem();
            mbar_arrive(tfull_bar(pend.stage));
            pend.advance(TS);
            cp_async_wait<0>();
            fence_proxy_async_smem();
            mbar_arrive(tfull_bar(pend.stage));
            pend.advance(TS);
#pragma unroll
            for (int i = 0; i < OMNI_TILE_N / 8; i++) off[i] = off_next[i];
        }
        cp_async_wait<0>();
    } else if (warp == 3 && lane == 0) {
        // ---------------------------------------------------------- token producer
        PipeState p, wr;
        const uint64_t pol_t = l2_policy_evict_last();
        int ready_group = -1;
        bool ok = true;
        while (ok) {
            ok = mbar_wait(ifull_bar(wr.stage), wr.phase, abort_flag, status);
            if (!ok) break;
            const int row0 = ring[wr.stage].row0, len = ring[wr.stage].len, expert = ring[wr.stage].expert;
            mbar_arrive(iempty_bar(wr.stage));
            wr.advance(RING);
            if (len < 0) break;
            if (ready && expert / group_size != ready_group) {
                // expert parallelism: this expert's rows are being written by other GPUs while the
                // kernel runs; wait (bounded, polling gently) until its whole group has arrived
                const int grp = expert / group_size;
                const uint32_t want = (uint32_t)__ldcg(need + grp);      // past L1, like the tile list
                const uint64_t t0 = globaltimer_ns();
                while (ld_acquire_sys_u32(ready + grp) != want) {
                    __nanosleep(500);
                    if (*abort_flag || globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
                        *abort_flag = 1;
                        atomicOr(status, OMNI_ST_TIMEOUT | OMNI_ST_TIMEOUT_ARRIVAL);
                        ok = false;
                        break;
                    }
                }
                if (!ok) break;
                fence_proxy_async_all();          // the rows are read next by TMA (async proxy)
                ready_group = grp;
            }
            const int bi = tok_box_index(len);
            const uint32_t bytes = (32u << bi) * (BK * 2);
            for (int ks = 0; ks < KSTAGES; ks++) {
                ok = mbar_wait(tempty_bar(p.stage), p.phase ^ 1u, abort_flag, status);
                if (!ok) break;
                armed_t[p.stage] = (int)p.phase;
                mbar_expect_tx(tfull_bar(p.stage), bytes);
                tma_load_2d_hint(tok_base + p.stage * T_TILE_BYTES, &tm_tok.m[bi], ks * BK, row0, tfull_bar(p.stage), pol_t);
                p.advance(TS);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------------------------------------------------- MMA issuer
        PipeState pw, pt, wr;
        bool ok = true;
        for (int it = 0; ok; it++) {
            ok = mbar_wait(ifull_bar(wr.stage), wr.phase, abort_flag, status);
            if (!ok) break;
            const int len = ring[wr.stage].len;
            mbar_arrive(iempty_bar(wr.stage));
            wr.advance(RING);
            if (len < 0) break;
            const int n_mma = (len + 15) & ~15;
            const uint32_t idesc = idesc_bf16(128, n_mma);
            const int buf = it % C::NBUF;
            const uint32_t use = (uint32_t)(it / C::NBUF);
            ok = mbar_wait(aempty_bar(buf), (use & 1u) ^ 1u, abort_flag, status);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d0 = tmem_base + (C::NBUF == 2 ? buf * 256 : 0);
            for (int ks = 0; ks < KSTAGES; ks++) {
                ok = mbar_wait(wfull_bar(pw.stage), pw.phase, abort_flag, status) &&
                     mbar_wait(tfull_bar(pt.stage), pt.phase, abort_flag, status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t sa = smem_base + pw.stage * W_BYTES;
                const uint64_t da0 = smem_desc_sw128(sa);
                const uint64_t db = smem_desc_sw128(tok_base + pt.stage * T_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < BK / 16; k++) {
                    const uint32_t acc = (ks | k) ? 1u : 0u;
                    umma_bf16(d0, da0 + 2u * k, db + 2u * k, idesc, acc);
                    if (C::NACC == 2)
                        umma_bf16(d0 + 256, smem_desc_sw128(sa + A_TILE_BYTES) + 2u * k, db + 2u * k, idesc, acc);
                }
                umma_commit(wempty_bar(pw.stage));   // both stages are free once these MMAs have read them
                umma_commit(tempty_bar(pt.stage));
                pw.advance(WS);
                pt.advance(TS);
            }
            if (!ok) break;
            umma_commit(afull_bar(buf));             // accumulator complete
        }
        // Whatever happened, wait (bounded) until every MMA issued by this thread retired
        // before TMEM is released.
        umma_commit(drain_bar);
        {
            const uint64_t t0 = globaltimer_ns();
            while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < WAIT_LIMIT_NS) {}
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------- epilogue: TMEM -> registers -> HBM
        const int q = warp & 3;                       // TMEM lane quadrant this warp may read
        const int half = (warp - 4) >> 2;             // two warps per quadrant split the column chunks
        PipeState wr;
        bool ok = true;
        for (int it = 0; ok; it++) {
            ok = mbar_wait(ifull_bar(wr.stage), wr.phase, abort_flag, status);
            if (!ok) break;
            const int row0 = ring[wr.stage].row0, len = ring[wr.stage].len, m = ring[wr.stage].m, expert = ring[wr.stage].expert;
            __syncwarp();
            if (lane == 0) mbar_arrive(iempty_bar(wr.stage));
            wr.advance(RING);
            if (len < 0) break;
            const int buf = it % C::NBUF;
            const uint32_t use = (uint32_t)(it / C::NBUF);
            ok = mbar_wait(afull_bar(buf), use & 1u, abort_flag, status);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + (C::NBUF == 2 ? buf * 256 : 0);
            const int nchunk = (len + 31) >> 5;
            const int col_out = m * 128 + q * 32 + lane;            // output column owned by this thread
            __nv_bfloat16 *orow = out + (long)row0 * C::OUT_COLS + col_out;
            if (MODE == MODE_GATEUP) {
                // SwiGLU into registers first, so that TMEM is handed back to the MMA warp
                // before the (slow, strided) stores to HBM start.
                uint32_t hp[4][16];
#pragma unroll
                for (int ci = 0; ci < 4; ci++) {
                    const int c = half + 2 * ci;
                    if (c < nchunk) {
                        uint32_t g[32], u[32];
                        tmem_ld32(t0 + c * 32, g);
                        tmem_ld32(t0 + 256 + c * 32, u);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const __nv_bfloat162 v = __floats2bfloat162_rn(
                                silu_mul(__uint_as_float(g[2 * j]), __uint_as_float(u[2 * j])),
                                silu_mul(__uint_as_float(g[2 * j + 1]), __uint_as_float(u[2 * j + 1])));
                            hp[ci][j] = *reinterpret_cast<const uint32_t *>(&v);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(aempty_bar(buf));
                unsigned short *o16 = reinterpret_cast<unsigned short *>(orow);
#pragma unroll
                for (int ci = 0; ci < 4; ci++) {
                    const int c = half + 2 * ci;
                    if (c < nchunk) {
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const int col = c * 32 + 2 * j;
                            if (col < len) o16[(long)col * C::OUT_COLS] = (unsigned short)(hp[ci][j] & 0xffffu);
                            if (col + 1 < len) o16[(long)(col + 1) * C::OUT_COLS] = (unsigned short)(hp[ci][j] >> 16);
                        }
                    }
                }
                if (done) {
                    // this warp's part of the expert's rows is out: tell the down kernel chained behind
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) atomicAdd(done + expert, 1);
                }
            } else {
                for (int c = half; c < nchunk; c += 2) {
                    uint32_t g[32];
                    tmem_ld32(t0 + c * 32, g);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int col = c * 32 + j;
                        if (col < len) orow[(long)col * C::OUT_COLS] = __float2bfloat16(__uint_as_float(g[j]));
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(aempty_bar(buf));
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        // a wait ran out: give copies already in flight a bounded chance to land
        for (int s = 0; s < WS + TS; s++) {
            const int par = s < WS ? armed_w[s] : armed_t[s - WS];
            if (par < 0) continue;
            const uint32_t bar = s < WS ? wfull_bar(s) : tfull_bar(s - WS);
            const uint64_t t0 = globaltimer_ns();
            while (!mbar_try_wait(bar, (uint32_t)par) && globaltimer_ns() - t0 < 50000000ull) {}
        }
    }
    __syncthreads();
    if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace

// ====================================================================== launchers
extern "C" {

cudaError_t omni_sm100_configure(void) {
    cudaError_t e;
    e = cudaFuncSetAttribute(expert_gemm_kernel<MODE_GATEUP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             GemmSmem<MODE_GATEUP>::TOTAL_BYTES);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(expert_gemm_kernel<MODE_DOWN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             GemmSmem<MODE_DOWN>::TOTAL_BYTES);
    return e;
}

cudaError_t omni_launch_gateup_sm100(const CUtensorMap *tm_w, const CUtensorMap *tm_x4, const omni_sort_state st,
                                     void *h, const uint32_t *ready, const int32_t *need, int group_size,
                                     const void *gather_src, const int32_t *gather_rows, int early_dependents, int announce,
                                     int n_sm, cudaStream_t s) {
    TokMaps tok;
    for (int i = 0; i < 4; i++) tok.m[i] = tm_x4[i];
    return omni_launch_chain(expert_gemm_kernel<MODE_GATEUP>, dim3(n_sm), dim3(GEMM_THREADS), GemmSmem<MODE_GATEUP>::TOTAL_BYTES, s,
                             *tm_w, tok, st.ttiles, st.n_ttiles, st.sched, (__nv_bfloat16 *)h, st.status, ready, need,
                             group_size > 0 ? group_size : 1, nullptr, 0, (const __nv_bfloat16 *)gather_src, gather_rows,
                             early_dependents, announce ? st.done : (int32_t *)nullptr, 0);
}

cudaError_t omni_launch_down_sm100(const CUtensorMap *tm_w, const CUtensorMap *tm_h4, const omni_sort_state st,
                                   void *d, const int32_t *tile_bounds, int group, int early_dependents, int chained,
                                   int n_sm, cudaStream_t s) {
    TokMaps tok;
    for (int i = 0; i < 4; i++) tok.m[i] = tm_h4[i];
    chained = chained && st.done && st.done_need;
    return omni_launch_chain(expert_gemm_kernel<MODE_DOWN>, dim3(n_sm), dim3(GEMM_THREADS), GemmSmem<MODE_DOWN>::TOTAL_BYTES, s,
                             *tm_w, tok, st.ttiles_down && !tile_bounds ? st.ttiles_down : st.ttiles, st.n_ttiles,
                             st.sched + 1 + (tile_bounds ? group : 0), (__nv_bfloat16 *)d,
                             st.status, chained ? (const uint32_t *)st.done : (const uint32_t *)nullptr,
                             chained ? st.done_need : (const int32_t *)nullptr, 1, tile_bounds, group, (const __nv_bfloat16 *)nullptr,
                             (const int32_t *)nullptr, early_dependents, (int32_t *)nullptr, chained);
}

}  // extern "C"
