// The two grouped expert products of the Clef-Omni MoE block on pairs of SMs (sm_100a):
//   expert_pair_kernel<GATEUP>  per expert: h = silu(Xe Wg^T) * (Xe Wu^T), SwiGLU in the epilogue
//                               (reference: metal/clef.metal:2455-2492, omni_expert_gemm + omni_swiglu;
//                               on one GPU the token rows are fetched through the permutation
//                               here: metal/clef.metal:2445-2453, omni_gather)
//   expert_pair_kernel<DOWN>    per expert: d = He Wd^T            (clef.metal:2455-2482)
//
// Two CTAs of a cluster (two SMs) work on one item together: one tcgen05.mma.cta_group::2 of
// shape M = 256 weight rows x N <= 256 token rows.  Each CTA loads its own 128 weight rows and
// HALF of the token rows into its own shared memory (plain per-CTA TMA loads or 16-byte
// cp.async gathers); the tensor cores of the two SMs exchange the token halves themselves, so a
// token row crosses the L2 -> SM path once per 256 weight rows instead of once per 128.  Each
// CTA ends up with the accumulator of its own 128 weight rows (128 lanes x N columns of its
// tensor memory), twice buffered, so the epilogue of one item runs under the MMAs of the next.
//
// Gate/up: the 128 weight rows of a CTA are 64 gate rows and the 64 up rows of the same
// intermediate columns, interleaved row by row by a three-dimensional TMA box over the
// [gate rows; up rows] matrix of the expert.  Gate and up of one column then sit in neighbouring
// lanes of one accumulator and SwiGLU needs one lane exchange instead of a second accumulator.
//
// Epilogue: TMEM -> registers -> a row-major tile in shared memory -> whole 128- or 256-byte
// row pieces written with 16-byte stores.  With expert parallelism the down product writes each
// row piece straight into the buffer of the rank that owns the token (plain peer stores), so
// the way back travels under the product, tile by tile, and no separate copy kernel runs.
//
// The same code runs with CTAS = 1 (no cluster, tcgen05 cta_group::1).  No load anywhere uses
// the cluster-multicast form.  Every wait is bounded; when one runs out the CTA (and its peer)
// raise OMNI_ST_TIMEOUT, drain what they issued, free tensor memory and return.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <type_traits>

#include "omni_internal.h"
#include "omni_ep_dev.cuh"
#include "omni_pdl.cuh"
#include "omni_ptx.cuh"

namespace {

// ------------------------------------------------------------------ cluster-scope helpers
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on a barrier that may live in the peer CTA (shared::cluster address)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// The same with the default ordering (release at CTA scope): for arrivals that only say "done"
// -- a stage was consumed, copies into this CTA's own shared memory have landed -- and publish no
// data written through the generic proxy into another CTA.  A cluster-scope release costs
// hundreds of nanoseconds and these arrivals sit on the per-stage critical path.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, int a, int b, int c, int d) {
    asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}

// What a CTA needs to give up cleanly: its own flag, its peer's, the status word.
struct Abort {
    volatile int *flag;
    uint32_t peer_flag;          // shared::cluster address of the peer's flag; 0 without a peer
    uint32_t *status;
    __device__ __forceinline__ void raise(uint32_t bits) const {
        *flag = 1;
        if (peer_flag) st_cluster_u32(peer_flag, 1u);
        atomicOr(status, bits);
    }
};

// Bounded wait on a barrier of this CTA.  False: the limit ran out or someone in the pair gave up.
// CLUSTER: acquire at cluster scope, for the one hand-over whose data another CTA wrote with
// ordinary stores (the item ring); everything else is signalled by the asynchronous units.
template <bool CLUSTER>
__device__ __noinline__ bool xwait_slow(uint32_t bar, uint32_t parity, const Abort &ab) {
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
        for (int i = 0; i < 256; i++)
            if (CLUSTER ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity)) return true;
        if (*ab.flag) return false;
        if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) { ab.raise(OMNI_ST_TIMEOUT); return false; }
    }
}
template <bool CLUSTER>
__device__ __forceinline__ bool xwait_impl(uint32_t bar, uint32_t parity, const Abort &ab) {
    for (int i = 0; i < 64; i++)
        if (CLUSTER ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity)) return true;
    return xwait_slow<CLUSTER>(bar, parity, ab);
}
template <int CTAS>
__device__ __forceinline__ bool xwait(uint32_t bar, uint32_t parity, const Abort &ab) { return xwait_impl<false>(bar, parity, ab); }
template <int CTAS>
__device__ __forceinline__ bool xwait_item(uint32_t bar, uint32_t parity, const Abort &ab) { return xwait_impl<CTAS == 2>(bar, parity, ab); }

// TMA loads whose completion is signalled on a barrier of the pair's first CTA.  Each CTA
// issues its own loads into its own shared memory: nothing here is a multicast.
template <int CTAS>
__device__ __forceinline__ void xtma_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar, uint64_t policy) {
    if (CTAS == 2)
        asm volatile(
            "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
            ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "l"(policy) : "memory");
    else
        tma_load_2d_hint(dst, map, x, y, bar, policy);
}
template <int CTAS>
__device__ __forceinline__ void xtma_3d(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar, uint64_t policy) {
    if (CTAS == 2)
        asm volatile(
            "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
            ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z), "l"(policy) : "memory");
    else
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
            ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z), "l"(policy) : "memory");
}

template <int CTAS>
__device__ __forceinline__ void xtmem_alloc(uint32_t dst_smem, uint32_t cols) {
    if (CTAS == 2) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
        tmem_alloc(dst_smem, cols);
        tmem_relinquish();
    }
}
template <int CTAS>
__device__ __forceinline__ void xtmem_dealloc(uint32_t addr, uint32_t cols) {
    if (CTAS == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
    else tmem_dealloc(addr, cols);
}
// D[tmem] (+)= A[smem] . B[smem]^T.  With CTAS = 2 the instruction spans both SMs of the pair:
// A = 128 rows per CTA, B = N/2 rows per CTA, at the same shared-memory offsets in both.
template <int CTAS>
__device__ __forceinline__ void xmma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if (CTAS == 2)
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    else
        umma_bf16(d_tmem, a_desc, b_desc, idesc, accumulate);
}
// One arrival on the barrier at this offset in EVERY CTA of the pair once all MMAs issued so far
// by this thread have completed (a barrier signal to both CTAs, not a data transfer).
template <int CTAS>
__device__ __forceinline__ void xcommit(uint32_t bar) {
    if (CTAS == 2)
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                     ::"r"(bar), "h"((uint16_t)3) : "memory");
    else
        umma_commit(bar);
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ------------------------------------------------------------------ configuration
enum { X_GATEUP = 0, X_DOWN = 1,
       // the two dense projections of the attention half, run as "one expert" over all token rows:
       X_QKV = 2,      // P[T][5120] = xn[T][2048] . W_qkv^T, BF16 out
       X_OPROJ = 3 };  // x[T][2048] += A[T][4096] . W_out^T, added into the FP32 residual
#ifndef X_GU_WS
#define X_GU_WS 7
#define X_GU_TS 5
#endif
#ifndef X_DN_WS
#define X_DN_WS 6
#define X_DN_TS 4
#endif
#ifndef X_GATHER_LAG            /* stages between issuing a gathered stage and handing it to the MMA thread */
#define X_GATHER_LAG 3
#endif

// ROWS: accumulator rows (weight rows) of one CTA; OUTC: output columns one CTA produces;
// MT: such CTA-level weight tiles per expert.
template <int MODE> struct XMode;
template <> struct XMode<X_GATEUP> { static constexpr int KTOT = OMNI_H, OUTC = 64, MT = OMNI_F / 64, OUT_COLS = OMNI_F; };
template <> struct XMode<X_DOWN> { static constexpr int KTOT = OMNI_F, OUTC = 128, MT = OMNI_H / 128, OUT_COLS = OMNI_H; };
template <> struct XMode<X_QKV> { static constexpr int KTOT = OMNI_H, OUTC = 128, MT = OMNI_QKV / 128, OUT_COLS = OMNI_QKV; };
template <> struct XMode<X_OPROJ> { static constexpr int KTOT = OMNI_NH * OMNI_HD, OUTC = 128, MT = OMNI_H / 128, OUT_COLS = OMNI_H; };

template <int MODE, int CTAS> struct XCfg {
    using M = XMode<MODE>;
    static constexpr int TOK_ROWS = OMNI_TILE_N / CTAS;                 // token rows one CTA stages per K slab
    static constexpr int T_BYTES = TOK_ROWS * BK * 2;                   // 32 KiB or 16 KiB
    static constexpr int W_BYTES = A_TILE_BYTES;                        // 16 KiB: 128 weight rows
    static constexpr int STAGE_OUT_BYTES = OMNI_TILE_N * M::OUTC * 2;   // 32 KiB (gate/up) or 64 KiB (down)
    // ring depths (stages of 64 K elements): weights come from HBM, token rows mostly from L2
    static constexpr int WS = CTAS == 2 ? (MODE == X_GATEUP ? X_GU_WS : X_DN_WS) : 4;
    static constexpr int TS = CTAS == 2 ? (MODE == X_GATEUP ? X_GU_TS : X_DN_TS) : 3;
    static constexpr int RING_BYTES = WS * W_BYTES + TS * T_BYTES;
    static constexpr int TOTAL_BYTES = RING_BYTES + STAGE_OUT_BYTES + 1024 + 1024;
    static constexpr int ITEMS_PER_TILE = M::MT / CTAS;
};
static_assert(XCfg<X_QKV, 2>::TOTAL_BYTES <= 232448 && XCfg<X_OPROJ, 2>::TOTAL_BYTES <= 232448 &&
              XCfg<X_GATEUP, 1>::TOTAL_BYTES <= 232448 && XCfg<X_DOWN, 1>::TOTAL_BYTES <= 232448 &&
              XCfg<X_GATEUP, 2>::TOTAL_BYTES <= 232448 && XCfg<X_DOWN, 2>::TOTAL_BYTES <= 232448, "shared memory budget");

constexpr int X_THREADS = 384;      // warp 0 scheduler + weight loads, 1 MMA, 2 TMEM (2+3 gather), 3 token loads, 4..11 epilogue
constexpr int X_COPY_THREADS = 128; // with COPY: warps 12..15 move this rank's token rows to the other ranks
constexpr int X_EPI_WARPS = 8;
constexpr int X_GATHER_THREADS = 64;
constexpr int X_RING = 4;

struct XTokMaps { CUtensorMap m[4]; };

struct XArgs {
    const omni_ttile *ttiles;
    const int32_t *n_ttiles;
    int32_t *work_counter;
    __nv_bfloat16 *out;                 // h [rows][768], d [rows][2048] or the q|k|v projections [rows][5120]
    float *resid;                       // output projection: the FP32 residual stream it adds into
    uint32_t *status;
    // expert parallelism, overlap mode: rows of a group of experts may be read once ready[grp] == need[grp]
    const uint32_t *ready;
    const int32_t *need;
    int group_size;
    // gate/up on one GPU: token row i of the permuted order is row gather_rows[i] of gather_src
    const __nv_bfloat16 *gather_src;
    const int32_t *gather_rows;
    // expert parallelism (pe.world > 1).  Down: result row i goes to row (rowinfo[i] & 0xfffff) of
    // pe.dret[rowinfo[i] >> 20], the buffer of the rank the token came from.  Gate/up with copy
    // warps: the spare warps send this rank's token rows (row rowmap[r] of disp_src for permuted
    // row r) to the owners of their experts while the other warps compute.
    omni_ep_peers pe;
    const int32_t *rowinfo;
    omni_ep_send send;                  // what the copy warps send from
    int need_blocks;                    // > 0: an arrival counter is complete at this value (it counts sender blocks), else at need[group]
    int early_dependents;
};

struct WorkSlotX { int expert, row0, len, m; };

// silu(g) * u with silu(g) = g * sigmoid(g) = (g/2) * (1 + tanh(g/2)): one special-function
// instruction per element instead of two (exp and reciprocal).  tanh.approx.f32 is accurate to
// about 2^-11 absolute; the result is rounded to BF16 (2^-9 relative) right after.
__device__ __forceinline__ float silu_mul(float g, float u) {
    const float hg = 0.5f * g;
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(hg));
    return fmaf(hg, t, hg) * u;
}

// ====================================================================== the kernel
// Work distribution as in the single-CTA kernels: an expert-major list of token tiles, items
// (token tile, weight block) claimed one at a time from a device counter by the first CTA of the
// pair, which hands each decoded item to the consumers of BOTH CTAs through a small ring that
// exists in each CTA's shared memory.
template <int MODE, int CTAS, bool COPY>
__global__ void __launch_bounds__(X_THREADS + (COPY ? X_COPY_THREADS : 0), 1)
expert_pair_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ XTokMaps tm_tok, const __grid_constant__ XArgs a) {
    using C = XCfg<MODE, CTAS>;
    using M = XMode<MODE>;
    constexpr int KSTAGES = M::KTOT / BK;
    constexpr int WS = C::WS, TS = C::TS, MI = C::ITEMS_PER_TILE;
    constexpr bool PAIR = CTAS == 2;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *const smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t tok_base = smem_base + WS * C::W_BYTES;
    uint8_t *const out_tile = smem_gen + C::RING_BYTES;                               // [256][OUTC] bf16
    const uint32_t bar_base = smem_base + C::RING_BYTES + C::STAGE_OUT_BYTES;
    auto wfull_bar = [&](int s) { return bar_base + 8u * s; };
    auto wempty_bar = [&](int s) { return bar_base + 8u * (WS + s); };
    auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * WS + s); };
    auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * WS + TS + s); };
    auto afull_bar = [&](int b) { return bar_base + 8u * (2 * WS + 2 * TS + b); };
    auto aempty_bar = [&](int b) { return bar_base + 8u * (2 * WS + 2 * TS + 2 + b); };
    const uint32_t drain_bar = bar_base + 8u * (2 * WS + 2 * TS + 4);
    auto ifull_bar = [&](int r) { return bar_base + 8u * (2 * WS + 2 * TS + 5 + r); };
    auto iempty_bar = [&](int r) { return bar_base + 8u * (2 * WS + 2 * TS + 5 + X_RING + r); };
    constexpr int N_BARS = 2 * WS + 2 * TS + 5 + 2 * X_RING;
    constexpr int MISC_OFF = (N_BARS * 8 + 15) & ~15;            // the item ring is written with 16-byte stores
    static_assert(MISC_OFF + 16 + 64 + X_RING * 16 <= 1024, "barrier block");
    uint8_t *misc = smem_gen + C::RING_BYTES + C::STAGE_OUT_BYTES + MISC_OFF;
    const uint32_t misc_u32 = bar_base + MISC_OFF;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(misc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(misc + 4);
    volatile int *epi_quit = reinterpret_cast<volatile int *>(misc + 8);        // [2] a warp of this epilogue half gave up
    volatile int *armed_w = reinterpret_cast<volatile int *>(misc + 16);        // [8] parity armed per weight stage, -1 none
    volatile int *armed_t = reinterpret_cast<volatile int *>(misc + 16 + 32);   // [8] same for the token ring
    volatile WorkSlotX *ring = reinterpret_cast<volatile WorkSlotX *>(misc + 16 + 64);
    const uint32_t ring_u32 = misc_u32 + 16 + 64;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    const bool leader = rank == 0;
    const bool gathering = a.gather_src != nullptr;
    const Abort ab{abort_flag, PAIR ? mapa_u32(misc_u32 + 4, rank ^ 1u) : 0u, a.status};
    // a barrier of the pair's first CTA, as an address every CTA of the pair may signal
    auto lead = [&](uint32_t bar) { return PAIR ? mapa_u32(bar, 0) : bar; };
    auto arrive_lead = [&](uint32_t bar) { if (PAIR) mbar_arrive_remote(mapa_u32(bar, 0)); else mbar_arrive(bar); };

    if (threadIdx.x == 0) {
        const int tp = gathering ? 2 : 1;                       // arrivals of a CTA's token producer per item
        for (int s = 0; s < WS; s++) { mbar_init(wfull_bar(s), 1); mbar_init(wempty_bar(s), 1); }
        for (int s = 0; s < TS; s++) { mbar_init(tfull_bar(s), gathering ? X_GATHER_THREADS * CTAS : 1); mbar_init(tempty_bar(s), 1); }
        for (int s = 0; s < 8; s++) { armed_w[s] = -1; armed_t[s] = -1; }
        for (int b = 0; b < 2; b++) { mbar_init(afull_bar(b), 1); mbar_init(aempty_bar(b), X_EPI_WARPS * CTAS); }
        mbar_init(drain_bar, 1);
        // consumers of an item: token producer(s), MMA thread and epilogue warps of the first CTA;
        // weight producer, token producer(s) and epilogue warps of the second
        for (int r = 0; r < X_RING; r++) {
            mbar_init(ifull_bar(r), 1);
            mbar_init(iempty_bar(r), (tp + 1 + X_EPI_WARPS) + (PAIR ? 1 + tp + X_EPI_WARPS : 0));
        }
        *abort_flag = 0;
        epi_quit[0] = 0; epi_quit[1] = 0;
        fence_mbar_init();
        prefetch_tmap(&tm_w);
        for (int i = 0; i < 4; i++) prefetch_tmap(&tm_tok.m[i]);
    }
    // the peer's barriers must exist before anything of this CTA can signal them
    if (PAIR) cluster_sync_all(); else __syncthreads();
    if (warp == 2) xtmem_alloc<CTAS>(smem_u32((const void *)tmem_slot), 512);
    dep_wait();                 // everything above overlaps the tail of the previous kernel
    if (a.early_dependents) dep_launch();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int work_lo = 0;
    const int n_work = *a.n_ttiles * MI;

    // weight tile of CTA `rank` for block m of an expert, K slab ks
    auto load_weights = [&](uint32_t dst, int expert, int m, int ks, uint32_t bar, uint64_t pol) {
        const int m_cta = m * CTAS + (int)rank;
        if (MODE == X_GATEUP) xtma_3d<CTAS>(dst, &tm_w, ks * BK, 0, expert * (2 * OMNI_F) + m_cta * 64, bar, pol);
        else xtma_2d<CTAS>(dst, &tm_w, ks * BK, expert * M::OUT_COLS + m_cta * 128, bar, pol);
    };

    if (warp == 0 && lane == 0 && leader) {
        // ---------------------------------------------------------- scheduler + weight producer
        // Claiming and decoding an item costs an atomic and two dependent global loads; they are
        // software-pipelined behind the TMA issue loop (item i+1 is decoded and item i+2 claimed
        // while item i is being loaded).
        PipeState p, wr;
        const uint64_t pol_w1 = l2_policy_evict_first(), pol_keep = l2_policy_evict_last();
        auto lookup = [&](int w, int &m, int &cnt) {          // item -> (weight block m, tile-list index)
            const omni_ttile t0 = a.ttiles[w / MI];
            const int first = t0.group & 0xffff;
            cnt = t0.group >> 16;
            const int local = w - first * MI;
            m = local / cnt;
            return first + local % cnt;
        };
        int cur_m = 0, cur_cnt = 1;
        omni_ttile cur = omni_ttile{0, 0, -1, 0};
        int w0 = work_lo + atomicAdd(a.work_counter, 1);
        int w1 = work_lo + atomicAdd(a.work_counter, 1);
        if (w0 < n_work) cur = a.ttiles[lookup(w0, cur_m, cur_cnt)];
        for (;;) {
            if (!xwait<CTAS>(iempty_bar(wr.stage), wr.phase ^ 1u, ab)) break;
            const int len = cur.len < 0 ? -1 : cur.len;
            ring[wr.stage].expert = cur.expert; ring[wr.stage].row0 = cur.row0;
            ring[wr.stage].len = len; ring[wr.stage].m = cur_m;
            mbar_arrive(ifull_bar(wr.stage));
            if (PAIR) {
                st_cluster_v4(mapa_u32(ring_u32 + 16u * wr.stage, 1), cur.expert, cur.row0, len, cur_m);
                mbar_arrive_cluster(mapa_u32(ifull_bar(wr.stage), 1));
            }
            if (len < 0) break;                                // told the consumers to stop
            wr.advance(X_RING);
            const int w2 = work_lo + atomicAdd(a.work_counter, 1);
            const bool has_next = w1 < n_work;
            omni_ttile head = omni_ttile{0, 0, 0, 0};
            if (has_next) head = a.ttiles[w1 / MI];
            int nxt_m = 0, nxt_cnt = 1;
            // a weight tile is read once per token tile of its expert: keep it in L2 while the
            // expert's other token tiles (claimed by neighbouring pairs) still need it
            const uint64_t pol_w = cur_cnt > 1 ? pol_keep : pol_w1;
            omni_ttile nxt = omni_ttile{0, 0, -1, 0};
            bool ok = true;
            for (int ks = 0; ks < KSTAGES; ks++) {
                if (ks == KSTAGES / 4 && has_next) {
                    const int first = head.group & 0xffff;
                    nxt_cnt = head.group >> 16;
                    const int local = w1 - first * MI;
                    nxt_m = local / nxt_cnt;
                    nxt = a.ttiles[first + local % nxt_cnt];
                }
                ok = xwait<CTAS>(wempty_bar(p.stage), p.phase ^ 1u, ab);
                if (!ok) break;
                armed_w[p.stage] = (int)p.phase;
                mbar_expect_tx(wfull_bar(p.stage), CTAS * C::W_BYTES);       // this CTA's tile and the peer's
                load_weights(smem_base + p.stage * C::W_BYTES, cur.expert, cur_m, ks, lead(wfull_bar(p.stage)), pol_w);
                p.advance(WS);
            }
            if (!ok) break;
            cur = nxt; cur_m = nxt_m; cur_cnt = nxt_cnt;
            w1 = w2;
        }
    } else if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------- weight producer of the second CTA
        PipeState p, wr;
        const uint64_t pol_w = l2_policy_evict_first();
        bool ok = true;
        while (ok) {
            ok = xwait_item<CTAS>(ifull_bar(wr.stage), wr.phase, ab);
            if (!ok) break;
            const int expert = ring[wr.stage].expert, len = ring[wr.stage].len, m = ring[wr.stage].m;
            arrive_lead(iempty_bar(wr.stage));
            wr.advance(X_RING);
            if (len < 0) break;
            for (int ks = 0; ks < KSTAGES; ks++) {
                ok = xwait<CTAS>(wempty_bar(p.stage), p.phase ^ 1u, ab);
                if (!ok) break;
                load_weights(smem_base + p.stage * C::W_BYTES, expert, m, ks, lead(wfull_bar(p.stage)), pol_w);
                p.advance(WS);
            }
        }
    } else if ((warp == 2 || warp == 3) && gathering) {
        // ---------------------------------------------------------- token producer, gathering
        // 64 threads fetch this CTA's share of the tile's token rows through the permutation:
        // 16-byte asynchronous copies, eight threads per 128-byte row segment, stored in the
        // 128-byte-swizzled layout the MMA descriptors expect (chunk c of row r at c ^ (r & 7)
        // inside its 8-row group).  A stage is handed to the MMA thread two stages after it was
        // issued, once the copies have landed and are ordered before the tensor core's reads.
        constexpr int LAG = (CTAS == 2 && MODE == X_GATEUP) ? X_GATHER_LAG : 2;
        static_assert(TS > LAG, "token ring too short for the copy lag");
        constexpr int NR = C::TOK_ROWS / 8;
        const uint64_t pol_t = l2_policy_evict_last();
        const int gt = threadIdx.x - 64;
        const int c = gt & 7, rb = gt >> 3;
        const uint32_t dst_off = (uint32_t)(rb * 128 + ((c ^ rb) << 4));
        const char *src0 = reinterpret_cast<const char *>(a.gather_src) + c * 16;
        PipeState p, pend, wr;
        int off[NR], off_next[NR];
        int ready_group = -1;
        auto next_item = [&](int (&o)[NR]) -> int {
            if (!xwait_item<CTAS>(ifull_bar(wr.stage), wr.phase, ab)) return -1;
            const int row0 = ring[wr.stage].row0, len = ring[wr.stage].len, expert = ring[wr.stage].expert;
            __syncwarp();
            if (lane == 0) arrive_lead(iempty_bar(wr.stage));
            wr.advance(X_RING);
            if (a.ready && len >= 0) {
                // expert parallelism: the rows and the row map of this expert's group are written by
                // other GPUs while the kernel runs; they are complete once the arrival counters of
                // every group up to it are (a token row may have come with an earlier group)
                const int grp = expert / a.group_size;
                bool ok = true;
                while (ready_group < grp && ok) {
                    const int g2 = ready_group + 1;
                    if (lane == 0) {
                        const uint32_t want = a.need_blocks ? (uint32_t)a.need_blocks : (uint32_t)a.need[g2];
                        const uint64_t t0 = globaltimer_ns();
                        while (ld_acquire_sys_u32(a.ready + g2) != want) {
                            __nanosleep(200);
                            if (*abort_flag || globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
                                ab.raise(OMNI_ST_TIMEOUT | OMNI_ST_TIMEOUT_ARRIVAL);
                                ok = false;
                                break;
                            }
                        }
                    }
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    ready_group = g2;
                }
                if (!ok) return -1;
            }
            const int share = (((len + 15) & ~15) / CTAS);            // token rows of the tile each CTA stages
            const int first = (int)rank * share;
#pragma unroll
            for (int i = 0; i < NR; i++) {
                const int r = rb + 8 * i;
                o[i] = (r < share && first + r < len) ? __ldcv(a.gather_rows + row0 + first + r) * (OMNI_H * 2) : -1;
            }
            return len;
        };
        // hands the oldest stage still in flight to the MMA thread once at most `left` newer ones are
        auto hand_over = [&](auto left) {
            cp_async_wait<decltype(left)::value>();
            fence_proxy_async_smem();
            arrive_lead(tfull_bar(pend.stage));
            pend.advance(TS);
        };
        int len = next_item(off);
        while (len >= 0) {
            bool ok = true;
            for (int ks = 0; ks < KSTAGES; ks++) {
                // hand over before blocking on a free stage: the MMA thread must never wait for
                // this loop to issue further copies
                if (ks >= LAG) hand_over(std::integral_constant<int, LAG - 1>{});
                ok = xwait<CTAS>(tempty_bar(p.stage), p.phase ^ 1u, ab);
                if (!ok) break;
                const uint32_t sb = tok_base + p.stage * C::T_BYTES + dst_off;
                const char *src = src0 + ks * (BK * 2);
#pragma unroll
                for (int i = 0; i < NR; i++)
                    if (off[i] >= 0) cp_async16(sb + i * 1024, src + off[i], pol_t);
                cp_async_commit();
                p.advance(TS);
            }
            if (!ok) break;
            // the next item's row indices travel while the last stages of this one land
            len = next_item(off_next);
            static_assert(LAG >= 1 && LAG <= 6, "copy lag");
            if (LAG >= 6) hand_over(std::integral_constant<int, 5>{});
            if (LAG >= 5) hand_over(std::integral_constant<int, 4>{});
            if (LAG >= 4) hand_over(std::integral_constant<int, 3>{});
            if (LAG >= 3) hand_over(std::integral_constant<int, 2>{});
            if (LAG >= 2) hand_over(std::integral_constant<int, 1>{});
            hand_over(std::integral_constant<int, 0>{});
#pragma unroll
            for (int i = 0; i < NR; i++) off[i] = off_next[i];
        }
        cp_async_wait<0>();
    } else if (warp == 3 && lane == 0) {
        // ---------------------------------------------------------- token producer, TMA
        PipeState p, wr;
        const uint64_t pol_t = l2_policy_evict_last();
        int ready_group = -1;
        bool ok = true;
        while (ok) {
            ok = xwait_item<CTAS>(ifull_bar(wr.stage), wr.phase, ab);
            if (!ok) break;
            const int row0 = ring[wr.stage].row0, len = ring[wr.stage].len, expert = ring[wr.stage].expert;
            arrive_lead(iempty_bar(wr.stage));
            wr.advance(X_RING);
            if (len < 0) break;
            if (a.ready && expert / a.group_size != ready_group) {
                // expert parallelism: this expert's rows are being written by other GPUs while the
                // kernel runs; wait (bounded, polling gently) until its whole group has arrived
                const int grp = expert / a.group_size;
                const uint32_t want = a.need_blocks ? (uint32_t)a.need_blocks : (uint32_t)a.need[grp];
                const uint64_t t0 = globaltimer_ns();
                while (ld_acquire_sys_u32(a.ready + grp) != want) {
                    __nanosleep(500);
                    if (*abort_flag || globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
                        ab.raise(OMNI_ST_TIMEOUT | OMNI_ST_TIMEOUT_ARRIVAL);
                        ok = false;
                        break;
                    }
                }
                if (!ok) break;
                fence_proxy_async_all();          // the rows are read next by TMA (async proxy)
                ready_group = grp;
            }
            const int share = ((len + 15) & ~15) / CTAS;
            const int bi = tok_box_index(share);
            const uint32_t bytes = (32u << bi) * (BK * 2);
            for (int ks = 0; ks < KSTAGES; ks++) {
                ok = xwait<CTAS>(tempty_bar(p.stage), p.phase ^ 1u, ab);
                if (!ok) break;
                if (leader) {
                    armed_t[p.stage] = (int)p.phase;
                    mbar_expect_tx(tfull_bar(p.stage), CTAS * bytes);
                }
                xtma_2d<CTAS>(tok_base + p.stage * C::T_BYTES, &tm_tok.m[bi], ks * BK, row0 + (int)rank * share,
                              lead(tfull_bar(p.stage)), pol_t);
                p.advance(TS);
            }
        }
    } else if (warp == 1 && lane == 0 && leader) {
        // ---------------------------------------------------------- MMA issuer (first CTA of the pair)
        PipeState pw, pt, wr;
        bool ok = true;
        for (int it = 0; ok; it++) {
            ok = xwait_item<CTAS>(ifull_bar(wr.stage), wr.phase, ab);
            if (!ok) break;
            const int len = ring[wr.stage].len;
            mbar_arrive(iempty_bar(wr.stage));
            wr.advance(X_RING);
            if (len < 0) break;
            const int n_mma = (len + 15) & ~15;
            const uint32_t idesc = idesc_bf16(128 * CTAS, n_mma);
            const int buf = it & 1;
            const uint32_t use = (uint32_t)(it >> 1);
            ok = xwait<CTAS>(aempty_bar(buf), (use & 1u) ^ 1u, ab);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d0 = tmem_base + buf * 256;
            for (int ks = 0; ks < KSTAGES; ks++) {
                ok = xwait<CTAS>(wfull_bar(pw.stage), pw.phase, ab) && xwait<CTAS>(tfull_bar(pt.stage), pt.phase, ab);
                if (!ok) break;
                tc_fence_after();
                const uint64_t da = smem_desc_sw128(smem_base + pw.stage * C::W_BYTES);
                const uint64_t db = smem_desc_sw128(tok_base + pt.stage * C::T_BYTES);
#pragma unroll
                for (int k = 0; k < BK / 16; k++) xmma<CTAS>(d0, da + 2u * k, db + 2u * k, idesc, (ks | k) ? 1u : 0u);
                xcommit<CTAS>(wempty_bar(pw.stage));     // both stages are free (in both CTAs) once these MMAs have read them
                xcommit<CTAS>(tempty_bar(pt.stage));
                pw.advance(WS);
                pt.advance(TS);
            }
            if (!ok) break;
            xcommit<CTAS>(afull_bar(buf));               // accumulator complete, in both CTAs
        }
        // Whatever happened, wait (bounded) until every MMA issued by this thread retired
        // before tensor memory is released.
        xcommit<CTAS>(drain_bar);
        {
            const uint64_t t0 = globaltimer_ns();
            while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < WAIT_LIMIT_NS) {}
        }
    } else if (COPY && warp >= 12) {
        // ---------------------------------------------------------- dispatch of this rank's token rows
        // (expert parallelism): each token once per owner rank, plain peer stores into the owners'
        // receive buffers, group by group, each group announced on the owner's arrival counter --
        // which the token producers above, here and on the other ranks, wait for.  Virtual block =
        // the copy warps of one CTA.
        const int nvb = (int)gridDim.x - (int)gridDim.x % a.pe.world;
        if ((int)blockIdx.x < nvb)
            ep_dispatch_dedup(a.pe, a.send, (int)blockIdx.x, nvb, warp - 12, X_COPY_THREADS / 32, lane, threadIdx.x == X_THREADS,
                              [] { named_bar_sync(3, X_COPY_THREADS); });
    } else if (warp >= 4 && warp < 12) {
        // ---------------------------------------------------------- epilogue: TMEM -> registers -> shared -> HBM
        // Each half stages its token rows in its own 128 rows of the shared-memory tile (which rows
        // of an item fall to which half changes from item to item, and the halves do not wait for
        // one another).  The four warps of a half meet at a named barrier twice per item.  A warp whose wait ran
        // out must therefore not leave on its own: it marks the half as giving up, still joins the
        // first barrier, and all four leave together right after it.
        const int q = warp & 3;                       // TMEM lane quadrant this warp may read
        const int half = (warp - 4) >> 2;             // the two warps of a quadrant split the token rows
        const int th = ((warp - 4) & 3) * 32 + lane;  // thread index inside the half (0..127)
        unsigned short *const tile16 = reinterpret_cast<unsigned short *>(out_tile);
        PipeState wr;
        for (int it = 0;; it++) {
            int row0 = 0, len = 0, m = 0;
            bool got = xwait_item<CTAS>(ifull_bar(wr.stage), wr.phase, ab);
            if (got) {
                row0 = ring[wr.stage].row0; len = ring[wr.stage].len; m = ring[wr.stage].m;
                __syncwarp();
                if (lane == 0) arrive_lead(iempty_bar(wr.stage));
                wr.advance(X_RING);
            }
            const bool stop = got && len < 0;
            const int buf = it & 1;
            const int nchunk = (len + 31) >> 5;
            const int c_lo = half ? (nchunk + 1) >> 1 : 0, c_hi = half ? nchunk : (nchunk + 1) >> 1;
            if (got && !stop) got = xwait<CTAS>(afull_bar(buf), (uint32_t)(it >> 1) & 1u, ab);
            if (got && !stop) {
                tc_fence_after();
                const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256;
                for (int c = c_lo; c < c_hi; c++) {
                    uint32_t v[32];
                    tmem_ld32(t0 + c * 32, v);
                    tmem_ld_wait();
                    if (MODE == X_GATEUP) {
                        // lanes 2i / 2i+1 hold gate / up of intermediate column i of this quadrant's
                        // sixteen; the even lane finishes token row c*32+j, the odd one row c*32+j+1
                        const int col = q * 16 + (lane >> 1), odd = lane & 1;
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            const uint32_t send = odd ? v[j] : v[j + 1];
                            const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 1);
                            const float hv = odd ? silu_mul(__uint_as_float(recv), __uint_as_float(v[j + 1]))
                                                 : silu_mul(__uint_as_float(v[j]), __uint_as_float(recv));
                            tile16[(half * 128 + (c - c_lo) * 32 + j + odd) * M::OUTC + col] = __bfloat16_as_ushort(__float2bfloat16(hv));
                        }
                    } else if (MODE == X_OPROJ) {
                        // added into the FP32 residual: a warp's 32 lanes are 32 consecutive columns of one row
                        float *xr = a.resid + (long)(row0 + c * 32) * M::OUT_COLS + (m * CTAS + (int)rank) * M::OUTC + q * 32 + lane;
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (c * 32 + j < len) xr[(long)j * M::OUT_COLS] += __uint_as_float(v[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            tile16[(half * 128 + (c - c_lo) * 32 + j) * M::OUTC + q * 32 + lane] = __bfloat16_as_ushort(__float2bfloat16(__uint_as_float(v[j])));
                    }
                }
                // tensor memory goes back to the MMA thread before the stores to HBM start
                tc_fence_before();
                __syncwarp();
                if (lane == 0) arrive_lead(aempty_bar(buf));
            }
            if (!got) epi_quit[half] = 1;
            named_bar_sync(1 + half, 128);            // the four quadrants of this half have written their columns
            if (stop || epi_quit[half]) break;
            const int r_lo = c_lo * 32, r_hi = MODE == X_OPROJ ? 0 : min(len, c_hi * 32);    // the output projection has stored already
            constexpr int LANES_PER_ROW = M::OUTC * 2 / 16;              // 8 (gate/up) or 16 (down)
            const int sub = th % LANES_PER_ROW;
            const int m_cta = m * CTAS + (int)rank;
            for (int r = r_lo + th / LANES_PER_ROW; r < r_hi; r += 128 / LANES_PER_ROW) {
                const uint4 val = *reinterpret_cast<const uint4 *>(out_tile + (half * 128 + r - r_lo) * (M::OUTC * 2) + sub * 16);
                __nv_bfloat16 *dst_row;
                if (MODE == X_DOWN && a.rowinfo) {
                    const int info = __ldg(a.rowinfo + row0 + r);
                    dst_row = reinterpret_cast<__nv_bfloat16 *>(a.pe.dret[info >> 20]) + (long)(info & 0xfffff) * M::OUT_COLS;
                } else {
                    dst_row = a.out + (long)(row0 + r) * M::OUT_COLS;
                }
                *reinterpret_cast<uint4 *>(dst_row + m_cta * M::OUTC + sub * 8) = val;
            }
            named_bar_sync(1 + half, 128);            // the tile may be overwritten by the next item
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
    // neither CTA of a pair may leave while the other's MMAs can still read its shared memory
    if (PAIR) cluster_sync_all(); else __syncthreads();
    if (warp == 2) { tc_fence_after(); xtmem_dealloc<CTAS>(tmem_base, 512); }
}

}  // namespace

// ====================================================================== launchers
namespace {

template <int MODE, int CTAS, bool COPY>
cudaError_t launch_pair(const CUtensorMap *tm_w, const CUtensorMap *tm_tok4, const XArgs &args, int n_sm, cudaStream_t s) {
    XTokMaps tok;
    for (int i = 0; i < 4; i++) tok.m[i] = tm_tok4[i];
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(n_sm - n_sm % CTAS));
    cfg.blockDim = dim3(X_THREADS + (COPY ? X_COPY_THREADS : 0));
    cfg.dynamicSmemBytes = XCfg<MODE, CTAS>::TOTAL_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (CTAS == 2) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 2; attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = 1;
        n++;
    }
    if (omni_dependent_launch_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, expert_pair_kernel<MODE, CTAS, COPY>, *tm_w, tok, args);
}

template <int MODE, int CTAS, bool COPY>
cudaError_t set_smem() {
    return cudaFuncSetAttribute(expert_pair_kernel<MODE, CTAS, COPY>, cudaFuncAttributeMaxDynamicSharedMemorySize, XCfg<MODE, CTAS>::TOTAL_BYTES);
}

}  // namespace

extern "C" {

cudaError_t omni_expert_configure(void) {
    cudaError_t e;
    if ((e = set_smem<X_GATEUP, 1, false>()) != cudaSuccess) return e;
    if ((e = set_smem<X_GATEUP, 2, false>()) != cudaSuccess) return e;
    if ((e = set_smem<X_GATEUP, 1, true>()) != cudaSuccess) return e;
    if ((e = set_smem<X_GATEUP, 2, true>()) != cudaSuccess) return e;
    if ((e = set_smem<X_DOWN, 1, false>()) != cudaSuccess) return e;
    if ((e = set_smem<X_QKV, 2, false>()) != cudaSuccess) return e;
    if ((e = set_smem<X_OPROJ, 2, false>()) != cudaSuccess) return e;
    return set_smem<X_DOWN, 2, false>();
}

cudaError_t omni_launch_gateup_pair(int ctas, const CUtensorMap *tm_w3, const CUtensorMap *tm_x4, const omni_sort_state st,
                                    void *h, const uint32_t *ready, const int32_t *need, int group_size,
                                    const void *gather_src, const int32_t *gather_rows, const omni_ep_peers *dispatch_to,
                                    const omni_ep_send *send, int early_dependents, int n_sm, cudaStream_t s) {
    XArgs a = {};
    a.ttiles = st.ttiles; a.n_ttiles = st.n_ttiles; a.work_counter = st.sched; a.out = (__nv_bfloat16 *)h; a.status = st.status;
    a.ready = ready; a.need = need; a.group_size = group_size > 0 ? group_size : 1;
    a.gather_src = (const __nv_bfloat16 *)gather_src; a.gather_rows = gather_rows;
    a.early_dependents = early_dependents;
    if (dispatch_to) {
        const int grid = n_sm - n_sm % ctas;
        a.pe = *dispatch_to;
        a.send = *send;
        a.need_blocks = grid - grid % dispatch_to->world;       // every rank launches the same grid
        return ctas == 2 ? launch_pair<X_GATEUP, 2, true>(tm_w3, tm_x4, a, n_sm, s) : launch_pair<X_GATEUP, 1, true>(tm_w3, tm_x4, a, n_sm, s);
    }
    return ctas == 2 ? launch_pair<X_GATEUP, 2, false>(tm_w3, tm_x4, a, n_sm, s) : launch_pair<X_GATEUP, 1, false>(tm_w3, tm_x4, a, n_sm, s);
}

cudaError_t omni_launch_down_pair(int ctas, const CUtensorMap *tm_w, const CUtensorMap *tm_h4, const omni_sort_state st,
                                  void *d, const omni_ep_peers *return_to, const int32_t *rowinfo, int early_dependents, int n_sm,
                                  cudaStream_t s) {
    XArgs a = {};
    a.ttiles = st.ttiles; a.n_ttiles = st.n_ttiles; a.work_counter = st.sched + 1;
    a.out = (__nv_bfloat16 *)d; a.status = st.status; a.group_size = 1;
    if (return_to) { a.pe = *return_to; a.rowinfo = rowinfo; }
    a.early_dependents = early_dependents;
    return ctas == 2 ? launch_pair<X_DOWN, 2, false>(tm_w, tm_h4, a, n_sm, s) : launch_pair<X_DOWN, 1, false>(tm_w, tm_h4, a, n_sm, s);
}

// The dense projections of the attention half on the same kernel: `st` holds a tile list that cuts
// the T token rows into tiles of one "expert" (omni_launch_dense_tiles), tm_w is the weight matrix
// [OUT_COLS][K] with a 64 x 128 box, tm_tok4 the token operand with boxes of 32..256 rows.
cudaError_t omni_launch_dense_pair(int which, const CUtensorMap *tm_w, const CUtensorMap *tm_tok4, const omni_sort_state st,
                                   int32_t *work_counter, void *out_bf16, float *resid, int n_sm, cudaStream_t s) {
    XArgs a = {};
    a.ttiles = st.ttiles; a.n_ttiles = st.n_ttiles; a.work_counter = work_counter;
    a.out = (__nv_bfloat16 *)out_bf16; a.resid = resid; a.status = st.status; a.group_size = 1;
    a.early_dependents = 1;
    return which == 0 ? launch_pair<X_QKV, 2, false>(tm_w, tm_tok4, a, n_sm, s) : launch_pair<X_OPROJ, 2, false>(tm_w, tm_tok4, a, n_sm, s);
}

}  // extern "C"
