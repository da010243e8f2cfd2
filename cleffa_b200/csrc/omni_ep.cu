// Expert parallelism for the Clef-Omni MoE block over the GPUs of one NVLink/NVSwitch node.
//
// The reference is single-device; this stage has no counterpart there.  Experts are sharded in
// contiguous id ranges (E/G per GPU), tokens are data-parallel.  Instead of a library
// all-to-all, rows move by plain peer stores into buffers that every rank has mapped from every
// other rank, so the permutation and the transfer are one kernel each way:
//
//   counts   every rank writes its 128 per-expert counts into every peer's count table, then a
//            flag barrier; from the table each rank derives, with no further communication,
//            where its rows land on the owners (source-rank-major inside each expert = the
//            canonical global assignment order) and the owner derives its local tile list.
//   dispatch one warp per permuted row copies the token's 4 KiB activation row straight into
//            the owner's expert-major buffer and records (source rank, source row) beside it.
//   return   after the expert products the owner copies each result row back to the source
//            rank's buffer at the source's own permuted position, so the unchanged combine
//            kernel finds it through `slots`.
//
// Cross-GPU ordering uses one monotonically increasing epoch per barrier and system-scope
// release/acquire on flag words; every spin is bounded (2 s unless the host sets another limit) and reports OMNI_ST_TIMEOUT
// through the status word instead of hanging.  No TMA or multicast touches peer memory: remote
// rows land in local HBM first and the GEMM kernels read them from there.
#include <cuda_bf16.h>
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

// One block.  Every rank tells every peer "I reached epoch E", then waits until all peers
// said so.  Writes made by earlier kernels of this stream are ordered before the flag by the
// system-scope fence.
__device__ void flag_barrier(const omni_ep_peers &pe, uint32_t epoch, uint32_t *status, uint64_t limit_ns = SPIN_LIMIT_NS) {
    __threadfence_system();
    __syncthreads();
    const int t = threadIdx.x;
    if (t < pe.world) st_release_sys(pe.flags[t] + pe.rank, epoch);
    if (t < pe.world) {
        const uint32_t *mine = pe.flags[pe.rank] + t;
        const uint64_t t0 = now_ns();
        // epochs only grow; '>=' in wrap-safe form
        while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
            if (now_ns() - t0 > limit_ns) { atomicOr(status, OMNI_ST_TIMEOUT | OMNI_ST_TIMEOUT_BARRIER); break; }
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(128) ep_barrier_kernel(omni_ep_peers pe, uint32_t epoch, uint32_t *status, uint64_t limit_ns) {
    flag_barrier(pe, epoch, status, limit_ns ? limit_ns : SPIN_LIMIT_NS);
}

// Realignment of the ranks (clef_omni_ep_sync).  The barrier epochs are host counters that
// advance with every barrier a rank launches, so a rank whose pass failed on the host part-way
// is behind its peers from then on.  This barrier does not use them: every rank publishes the
// number of successful syncs it has seen plus one (`count`) and its current epoch, waits until
// every peer's count has reached its own, and then all adopt the largest epoch and the largest
// count they read.  A rank that waited alone keeps its old count on the host, so that its next
// attempt publishes the same number again and meets the others there.
__global__ void __launch_bounds__(32) ep_sync_kernel(omni_ep_peers pe, uint32_t count, uint32_t epoch, uint32_t *status,
                                                     uint32_t *result, uint64_t limit_ns) {
    const int t = threadIdx.x;
    __threadfence_system();
    if (t < pe.world) {
        st_release_sys(pe.flags[t] + OMNI_EP_SYNC_WORD + OMNI_EP_MAX + pe.rank, epoch);
        st_release_sys(pe.flags[t] + OMNI_EP_SYNC_WORD + pe.rank, count);
    }
    uint32_t c = count, e = epoch;
    bool ok = true;
    if (t < pe.world) {
        const uint32_t *mine = pe.flags[pe.rank] + OMNI_EP_SYNC_WORD;
        const uint64_t t0 = now_ns();
        while ((int32_t)((c = ld_acquire_sys(mine + t)) - count) < 0) {
            if (now_ns() - t0 > limit_ns) { atomicOr(status, OMNI_ST_TIMEOUT | OMNI_ST_TIMEOUT_BARRIER); ok = false; break; }
        }
        e = ld_acquire_sys(mine + OMNI_EP_MAX + t);
    }
    ok = __all_sync(0xffffffffu, ok);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const uint32_t oc = __shfl_xor_sync(0xffffffffu, c, s), oe = __shfl_xor_sync(0xffffffffu, e, s);
        if ((int32_t)(oc - c) > 0) c = oc;
        if ((int32_t)(oe - e) > 0) e = oe;
    }
    if (t == 0 && ok) { result[0] = c; result[1] = e; }
}

// Publish my counts, barrier, then plan.  One block of 128 threads, thread e = expert e.
__global__ void __launch_bounds__(OMNI_E) ep_plan_kernel(omni_ep_peers pe, uint32_t epoch, omni_sort_state st,
                                                         int32_t *send_base, int32_t *n_local_rows, int32_t *need,
                                                         int32_t *ret_bounds, uint64_t limit_ns) {
    __shared__ int tot[OMNI_E], scan[OMNI_E], tiles[OMNI_E];
    const int e = threadIdx.x;
    const int G = pe.world, EL = OMNI_E / G;
    const int mine = st.counts[e];
    for (int p = 0; p < G; p++) pe.counts[p][pe.rank * OMNI_E + e] = mine;
    // arrival counters of this rank's experts start at zero; peers add to them only after the barrier
    pe.flags[pe.rank][OMNI_EP_READY_WORD + e] = 0;
    flag_barrier(pe, epoch, st.status, limit_ns);
    // table[s][e] = rows rank s routes to expert e
    const int32_t *table = pe.counts[pe.rank];
    int total = 0, before_me = 0;
    for (int s = 0; s < G; s++) {
        const int c = __ldcv(table + s * OMNI_E + e);     // written by peers: bypass L1
        if (s < pe.rank) before_me += c;
        total += c;
    }
    tot[e] = total;
    __syncthreads();
    // Every rank holds the same table, so every rank can see an owner whose buffers would not
    // hold what is routed to it: the senders skip those rows, the owner returns nothing, and
    // each rank's own status word says so (its combine would otherwise read rows of an earlier pass).
    if (e < G) {
        int to_owner = 0;
        for (int o = e * EL; o < (e + 1) * EL; o++) to_owner += tot[o];
        if (to_owner > OMNI_ROWS) atomicOr(st.status, OMNI_ST_EP_OVERFLOW);
    }
    // base of expert e inside its owner's buffer: totals of the owner's earlier experts
    const int owner = e / EL, first = owner * EL;
    int base = 0;
    for (int o = first; o < e; o++) base += tot[o];
    send_base[e] = base + before_me;
    // the owner's view: local experts first..first+EL-1 of THIS rank
    const int le = e;                       // threads 0..EL-1 act for local expert le
    int n = 0, nt = 0;
    if (le < EL) { n = tot[pe.rank * EL + le]; nt = (n + OMNI_TILE_N - 1) / OMNI_TILE_N; }
    scan[e] = n; tiles[e] = nt;
    __syncthreads();
    if (e == 0) {                           // EL <= 128: a serial scan over the local experts is short
        int rows = 0, t = 0;
        for (int l = 0; l < EL; l++) { const int c = scan[l], k = tiles[l]; scan[l] = rows; tiles[l] = t; rows += c; t += k; }
        // rows each arrival group of local experts must receive before its rows may be read
        const int gsz = omni_ep_group_size(G);
        for (int grp = 0; grp * gsz < EL; grp++) {
            const int hi = min((grp + 1) * gsz, EL);
            need[grp] = (hi < EL ? scan[hi] : rows) - scan[grp * gsz];
        }
        // the down product and the way back run in RET_GROUPS groups of local experts
        for (int rg = 0; rg <= OMNI_EP_RET_GROUPS; rg++) {
            const int le0 = min(EL, (EL * rg + OMNI_EP_RET_GROUPS - 1) / OMNI_EP_RET_GROUPS);
            ret_bounds[rg] = le0 < EL ? tiles[le0] : t;
            ret_bounds[OMNI_EP_RET_GROUPS + 1 + rg] = le0 < EL ? scan[le0] : rows;
        }
        *n_local_rows = rows;
        *st.n_ttiles = rows <= OMNI_ROWS ? t : 0;
        for (int i = 0; i < 8; i++) st.sched[i] = 0;
        if (rows > OMNI_ROWS) atomicOr(st.status, OMNI_ST_EP_OVERFLOW);
    }
    __syncthreads();
    if (le < EL && *n_local_rows <= OMNI_ROWS) {
        const int off = scan[le], firstt = tiles[le];
        const int base = nt ? n / nt : 0, extra = nt ? n % nt : 0;      // near-equal tiles, as in assign_scan_kernel
        for (int j = 0; j < nt; j++)
            st.ttiles[firstt + j] = omni_ttile{le, off + j * base + min(j, extra), base + (j < extra), firstt | (nt << 16)};
    }
}

// One warp per permuted row of this rank: 4 KiB to the owner's buffer + its origin tag.
// Blocks are dealt round-robin to destination ranks, starting with the next rank, so that at
// every moment each rank writes to all owners at once and no owner is the target of everyone
// (walking the rows in expert order would make all ranks hit owner 0 first, then owner 1, ...:
// measured 2.6x slower on 8 GPUs).  An owner's experts are sent in ascending groups; after each
// group the block adds the number of rows it delivered to the owner's arrival counter of that
// group (one system-scope release per block and group), which is what the owner's gate/up
// kernel waits on before it reads those rows.
template <bool SIGNAL>
__global__ void __launch_bounds__(256) ep_dispatch_kernel(omni_ep_peers pe, const uint4 *__restrict__ xn,
                                                          const int32_t *__restrict__ rowmap,
                                                          const int32_t *__restrict__ offsets,
                                                          const int32_t *__restrict__ send_base) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // without SIGNAL (phases separated by a barrier) the owner's experts form one group and nothing is announced
    const int G = pe.world, EL = OMNI_E / G, gsz = SIGNAL ? omni_ep_group_size(G) : EL;
    const int owner = (int)((blockIdx.x % G + pe.rank + 1) % G);
    const int sub = blockIdx.x / G, nsub = (gridDim.x - (blockIdx.x % G) + G - 1) / G;   // blocks serving this owner
    uint4 *xg = reinterpret_cast<uint4 *>(pe.xg[owner]);
    int32_t *info = pe.rowinfo[owner];
    uint32_t *arrived = pe.flags[owner] + OMNI_EP_READY_WORD;        // the owner's per-group arrival counters
    int e = owner * EL;
    for (int grp = 0; grp * gsz < EL; grp++) {
        const int lo = offsets[owner * EL + grp * gsz], hi = offsets[owner * EL + min((grp + 1) * gsz, EL)];
        for (int r = lo + sub * 8 + warp; r < hi; r += nsub * 8) {
            while (offsets[e + 1] <= r) e++;                        // rows ascend: the expert only moves forward
            const long dst = (long)send_base[e] + (r - offsets[e]);
            if (dst >= OMNI_ROWS) continue;                         // owner overflow: flagged by its plan kernel
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
        __syncthreads();
        if (threadIdx.x == 0) {
            // rows of [lo, hi) that fell to this block: positions j with (j / 8) % nsub == sub
            const int n = hi - lo, full = n / (nsub * 8), rem = n % (nsub * 8);
            const int mine = full * 8 + max(0, min(8, rem - sub * 8));
            if (mine) red_release_sys_add(arrived + grp, (uint32_t)mine);
        }
    }
}

// One warp per local expert-major row: result row back to the source rank's permuted position.
__global__ void __launch_bounds__(256) ep_return_kernel(omni_ep_peers pe, const uint4 *__restrict__ d,
                                                        const int32_t *__restrict__ rowinfo,
                                                        const int32_t *__restrict__ row_bounds, int group, int group_end) {
    const int lane = threadIdx.x & 31;
    const int warps = gridDim.x * 8;
    const int first = row_bounds[group];
    int n = row_bounds[group_end];
    if (n > OMNI_ROWS) n = 0;
    for (int r = first + blockIdx.x * 8 + (threadIdx.x >> 5); r < n; r += warps) {
        const int info = rowinfo[r];
        const int src_rank = info >> 20, src_row = info & 0xfffff;
        const uint4 *src = d + (long)r * (OMNI_H / 8);
        uint4 *out = reinterpret_cast<uint4 *>(pe.dret[src_rank]) + (long)src_row * (OMNI_H / 8);
        uint4 v[8];
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = src[lane + 32 * i];
#pragma unroll
        for (int i = 0; i < 8; i++) out[lane + 32 * i] = v[i];
    }
}

}  // namespace

extern "C" {

cudaError_t omni_launch_ep_plan(const omni_ep_peers *pe, uint32_t epoch, omni_sort_state st, int32_t *send_base,
                                int32_t *n_local_rows, int32_t *need, int32_t *ret_bounds, uint64_t limit_ns, cudaStream_t s) {
    ep_plan_kernel<<<1, OMNI_E, 0, s>>>(*pe, epoch, st, send_base, n_local_rows, need, ret_bounds, limit_ns ? limit_ns : SPIN_LIMIT_NS);
    return cudaGetLastError();
}

cudaError_t omni_launch_ep_barrier(const omni_ep_peers *pe, uint32_t epoch, uint32_t *status, uint64_t limit_ns,
                                   cudaStream_t s) {
    ep_barrier_kernel<<<1, 128, 0, s>>>(*pe, epoch, status, limit_ns);
    return cudaGetLastError();
}

cudaError_t omni_launch_ep_sync(const omni_ep_peers *pe, uint32_t count, uint32_t epoch, uint32_t *status, uint32_t *result,
                                uint64_t limit_ns, cudaStream_t s) {
    ep_sync_kernel<<<1, 32, 0, s>>>(*pe, count, epoch, status, result, limit_ns ? limit_ns : SPIN_LIMIT_NS);
    return cudaGetLastError();
}

cudaError_t omni_launch_ep_dispatch(const omni_ep_peers *pe, const void *xn, const int32_t *rowmap, const int32_t *offsets,
                                    const int32_t *send_base, int rows8, int signal, int n_sm, cudaStream_t s) {
    // One block per SM at most: the copy is bound by NVLink, not by parallelism, and a small
    // footprint (256 threads x 32 registers) lets it share SMs with a running expert-product
    // kernel of another micro-batch instead of waiting for it.
    (void)rows8;
    int blocks = n_sm - n_sm % pe->world;                // the same number of blocks for every owner
    if (blocks < pe->world) blocks = pe->world;
    if (signal) ep_dispatch_kernel<true><<<blocks, 256, 0, s>>>(*pe, (const uint4 *)xn, rowmap, offsets, send_base);
    else ep_dispatch_kernel<false><<<blocks, 256, 0, s>>>(*pe, (const uint4 *)xn, rowmap, offsets, send_base);
    return cudaGetLastError();
}

cudaError_t omni_launch_ep_return(const omni_ep_peers *pe, const void *d, const int32_t *rowinfo,
                                  const int32_t *row_bounds, int group, int group_end, int n_sm, cudaStream_t s) {
    ep_return_kernel<<<n_sm, 256, 0, s>>>(*pe, (const uint4 *)d, rowinfo, row_bounds, group, group_end);
    return cudaGetLastError();
}

}  // extern "C"
