// Device-side pieces of the expert-parallel exchange that more than one kernel uses: system-scope
// flag operations and the dispatch of this rank's token rows to the ranks that own their experts
// (run by a copy kernel of its own, or by the spare warps of the gate/up expert kernel so that
// the transfer travels under the product).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "omni_internal.h"

namespace {

constexpr uint64_t SPIN_LIMIT_NS = 2000000000ull;      // 2 s: every legitimate wait is far shorter

__device__ __forceinline__ uint64_t now_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Adds to a counter in (possibly another GPU's) memory; every store this warp made before the
// preceding __syncwarp is visible to whoever acquires the new value.
__device__ __forceinline__ void red_release_sys_add(uint32_t *p, uint32_t v) {
    __threadfence_system();
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One warp per permuted row of this rank: 4 KiB to the owner's buffer + its origin tag.
// The copying threads form `nvb` virtual blocks of `nwarp` warps; block `vb` serves one owner.
// Blocks are dealt round-robin to destination ranks, starting with the next rank, so that at
// every moment each rank writes to all owners at once and no owner is the target of everyone
// (walking the rows in expert order would make all ranks hit owner 0 first, then owner 1, ...:
// measured 2.6x slower on 8 GPUs).  With SIGNAL an owner's experts are sent in ascending groups;
// after each group the block adds the number of rows it delivered to the owner's arrival counter
// of that group (one system-scope release per block and group), which is what the owner's
// gate/up kernel waits on before it reads those rows.  `sync` is a barrier over the block's
// threads; `first` is true in exactly one of them.  nvb must be a multiple of the world size.
template <bool SIGNAL, typename Sync>
__device__ __forceinline__ void ep_dispatch_rows(const omni_ep_peers &pe, const uint4 *__restrict__ xn,
                                                 const int32_t *__restrict__ rowmap, const int32_t *__restrict__ offsets,
                                                 const int32_t *__restrict__ send_base, int vb, int nvb, int warp, int nwarp,
                                                 int lane, bool first, Sync sync) {
    // without SIGNAL (phases separated by a barrier) the owner's experts form one group and nothing is announced
    const int G = pe.world, EL = OMNI_E / G, gsz = SIGNAL ? omni_ep_group_size(G) : EL;
    const int owner = (vb % G + pe.rank + 1) % G;
    const int sub = vb / G, nsub = nvb / G;                       // blocks serving this owner
    uint4 *xg = reinterpret_cast<uint4 *>(pe.xg[owner]);
    int32_t *info = pe.rowinfo[owner];
    uint32_t *arrived = pe.flags[owner] + OMNI_EP_READY_WORD;        // the owner's per-group arrival counters
    int e = owner * EL;
    for (int grp = 0; grp * gsz < EL; grp++) {
        const int lo = offsets[owner * EL + grp * gsz], hi = offsets[owner * EL + min((grp + 1) * gsz, EL)];
        for (int r = lo + sub * nwarp + warp; r < hi; r += nsub * nwarp) {
            while (offsets[e + 1] <= r) e++;                        // rows ascend: the expert only moves forward
            const long dst = (long)send_base[e] + (r - offsets[e]);
            if (dst >= OMNI_ROWS) continue;                         // owner overflow: flagged by the plan kernel
            const uint4 *src = xn + (long)rowmap[r] * (OMNI_H / 8);
            uint4 *out = xg + dst * (OMNI_H / 8);
            uint4 v[8];
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = __ldg(src + lane + 32 * i);
#pragma unroll
            for (int i = 0; i < 8; i++) out[lane + 32 * i] = v[i];
            if (lane == 0) info[dst] = (pe.rank << 20) | r;
        }
        if (!SIGNAL) break;
        __threadfence_system();          // every thread: its own row stores are out before the count is published
        sync();
        if (first) {
            // rows of [lo, hi) that fell to this block: positions j with (j / nwarp) % nsub == sub
            const int n = hi - lo, full = n / (nsub * nwarp), rem = n % (nsub * nwarp);
            const int mine = full * nwarp + max(0, min(nwarp, rem - sub * nwarp));
            if (mine) red_release_sys_add(arrived + grp, (uint32_t)mine);
        }
    }
}

// The de-duplicated dispatch.  A token row is sent ONCE to every rank that owns at least one of
// its experts (4.6 instead of 7 remote copies per token on 8 GPUs), into that owner's receive
// buffer; which received row an expert-major row of the owner reads is told by a row map the
// senders fill beside the origin tags.  A token belongs to the bucket (owner, first group of the
// owner's experts that needs it); buckets are sent in ascending groups, and so are the row-map
// entries of each group's experts, so that the owner's gate/up kernel may start on group g once
// the arrival counters of groups 0..g are complete.  A counter counts sender BLOCKS (every
// block adds one per group, after a system-scope fence over its stores), so its target is the
// same number on every rank: nvb, the number of virtual blocks of a sender, which is why every
// rank must launch the same grid.
template <typename Sync>
__device__ __forceinline__ void ep_dispatch_dedup(const omni_ep_peers &pe, const omni_ep_send &sd, int vb, int nvb, int warp,
                                                  int nwarp, int lane, bool first, Sync sync) {
    const int G = pe.world, EL = OMNI_E / G, gsz = omni_ep_group_size(G);
    const int owner = (vb % G + pe.rank + 1) % G;
    const int sub = vb / G, nsub = nvb / G;                       // blocks serving this owner
    uint4 *xr = reinterpret_cast<uint4 *>(pe.xg[owner]);
    int32_t *info = pe.rowinfo[owner], *grow = pe.grow[owner];
    uint32_t *arrived = pe.flags[owner] + OMNI_EP_READY_WORD;
    const uint4 *xn = reinterpret_cast<const uint4 *>(sd.xn);
    for (int grp = 0; grp * gsz < EL; grp++) {
        const int b = owner * OMNI_EP_GROUPS + grp;
        // the token rows of this bucket: one warp per row
        const int n = sd.send_cnt[b];
        const long base = sd.recv_base[b];
        const int32_t *list = sd.bucket_list + (long)b * OMNI_CHUNK;
        for (int p = sub * nwarp + warp; p < n; p += nsub * nwarp) {
            if (base + p >= OMNI_ROWS) continue;                    // owner overflow: flagged by the plan kernel
            const uint4 *src = xn + (long)list[p] * (OMNI_H / 8);
            uint4 *out = xr + (base + p) * (OMNI_H / 8);
            uint4 v[8];
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = __ldg(src + lane + 32 * i);
#pragma unroll
            for (int i = 0; i < 8; i++) out[lane + 32 * i] = v[i];
        }
        // the expert-major rows of this group's experts: origin tag and received row, one thread per row
        const int e_lo = owner * EL + grp * gsz, e_hi = owner * EL + min((grp + 1) * gsz, EL);
        const int lo = sd.offsets[e_lo], hi = sd.offsets[e_hi];
        int e = e_lo;
        for (int r = lo + (sub * nwarp + warp) * 32 + lane; r < hi; r += nsub * nwarp * 32) {
            while (sd.offsets[e + 1] <= r) e++;                     // rows ascend: the expert only moves forward
            const long dst = (long)sd.send_base[e] + (r - sd.offsets[e]);
            if (dst >= OMNI_ROWS) continue;
            const int slot = sd.tok_slot[sd.rowmap[r] * OMNI_EP_MAX + owner];
            info[dst] = (pe.rank << 20) | r;
            grow[dst] = sd.recv_base[owner * OMNI_EP_GROUPS + (slot >> 24)] + (slot & 0xffffff);
        }
        __threadfence_system();          // every thread: its stores are out before the block is counted
        sync();
        if (first) red_release_sys_add(arrived + grp, 1u);
    }
}

}  // namespace
