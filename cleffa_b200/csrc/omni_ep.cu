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
#include "omni_ep_dev.cuh"
#include "omni_pdl.cuh"

namespace {

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
    dep_wait();                 // part of the pass's dependent-launch chain: resident early, works only after the down kernel
    dep_launch();
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

// Tokens -> buckets of the de-duplicated dispatch.  One thread per token: for every owner rank
// the first (lowest) group of that owner's experts among the token's eight; the token takes the
// next free position of the bucket (owner, group).  Positions are handed out by atomics, so the
// order inside a bucket differs from run to run; it only names rows of the receive buffer.
__global__ void __launch_bounds__(256) ep_bucket_kernel(const int32_t *__restrict__ ids, int T, int world,
                                                        int32_t *__restrict__ tok_slot, int32_t *__restrict__ bucket_cnt,
                                                        int32_t *__restrict__ bucket_list) {
    dep_wait();
    dep_launch();
    const int t = blockIdx.x * 256 + threadIdx.x;
    if (t >= T) return;
    const int EL = OMNI_E / world, gsz = omni_ep_group_size(world);
    const int4 a = *reinterpret_cast<const int4 *>(ids + (long)t * 8), b = *reinterpret_cast<const int4 *>(ids + (long)t * 8 + 4);
    const int id[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int o = 0; o < OMNI_EP_MAX; o++) {
        int g = OMNI_EP_GROUPS;
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int e = id[k] & (OMNI_E - 1);
            if (e / EL == o) g = min(g, (e % EL) / gsz);
        }
        int slot = -1;
        if (g < OMNI_EP_GROUPS) {
            const int bkt = o * OMNI_EP_GROUPS + g;
            const int pos = atomicAdd(bucket_cnt + bkt, 1);
            bucket_list[(long)bkt * OMNI_CHUNK + pos] = t;
            slot = (g << 24) | pos;
        }
        tok_slot[(long)t * OMNI_EP_MAX + o] = slot;
    }
}

// Publish my counts, barrier, then plan.  One block of 128 threads, thread e = expert e.
__global__ void __launch_bounds__(OMNI_E) ep_plan_kernel(omni_ep_peers pe, uint32_t epoch, omni_sort_state st,
                                                         int32_t *send_base, int32_t *n_local_rows, int32_t *need,
                                                         int32_t *bucket_cnt, int32_t *send_cnt, int32_t *recv_base,
                                                         uint64_t limit_ns) {
    __shared__ int tot[OMNI_E], scan[OMNI_E], tiles[OMNI_E];
    dep_wait();
    dep_launch();
    const int e = threadIdx.x;
    const int G = pe.world, EL = OMNI_E / G;
    const int mine = st.counts[e];
    for (int p = 0; p < G; p++) pe.counts[p][pe.rank * OMNI_EP_COUNT_STRIDE + e] = mine;
    // and, for the de-duplicated dispatch, how many tokens it sends per (owner, group) bucket; the
    // counter is left at zero for the next pass
    if (e < OMNI_EP_BUCKETS) {
        const int c = bucket_cnt[e];
        send_cnt[e] = c;
        bucket_cnt[e] = 0;
        for (int p = 0; p < G; p++) pe.counts[p][pe.rank * OMNI_EP_COUNT_STRIDE + OMNI_E + e] = c;
    }
    // arrival counters of this rank's experts start at zero; peers add to them only after the barrier
    pe.flags[pe.rank][OMNI_EP_READY_WORD + e] = 0;
    flag_barrier(pe, epoch, st.status, limit_ns);
    // table[s][e] = rows rank s routes to expert e
    const int32_t *table = pe.counts[pe.rank];
    int total = 0, before_me = 0;
    for (int s = 0; s < G; s++) {
        const int c = __ldcv(table + s * OMNI_EP_COUNT_STRIDE + e);     // written by peers: bypass L1
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
    // bucket (owner o, group g): this rank's tokens follow those of lower groups from every rank
    // and those of this group from lower ranks in the owner's receive buffer
    if (e < OMNI_EP_BUCKETS) {
        const int o = e / OMNI_EP_GROUPS, g = e % OMNI_EP_GROUPS;
        int base = 0, all = 0;
        for (int s = 0; s < G; s++)
            for (int gg = 0; gg < OMNI_EP_GROUPS; gg++) {
                const int c = __ldcv(table + s * OMNI_EP_COUNT_STRIDE + OMNI_E + o * OMNI_EP_GROUPS + gg);
                all += c;
                if (gg < g || (gg == g && s < pe.rank)) base += c;
            }
        recv_base[e] = base;
        if (o < G && all > OMNI_ROWS) atomicOr(st.status, OMNI_ST_EP_OVERFLOW);
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

template <bool SIGNAL>
__global__ void __launch_bounds__(256) ep_dispatch_kernel(omni_ep_peers pe, const uint4 *__restrict__ xn,
                                                          const int32_t *__restrict__ rowmap,
                                                          const int32_t *__restrict__ offsets,
                                                          const int32_t *__restrict__ send_base) {
    ep_dispatch_rows<SIGNAL>(pe, xn, rowmap, offsets, send_base, (int)blockIdx.x, (int)gridDim.x, threadIdx.x >> 5, 8,
                             threadIdx.x & 31, threadIdx.x == 0, [] { __syncthreads(); });
}

}  // namespace

extern "C" {

cudaError_t omni_launch_ep_plan(const omni_ep_peers *pe, uint32_t epoch, omni_sort_state st, int32_t *send_base,
                                int32_t *n_local_rows, int32_t *need, int32_t *bucket_cnt, int32_t *send_cnt, int32_t *recv_base,
                                uint64_t limit_ns, cudaStream_t s) {
    return omni_launch_chain(ep_plan_kernel, dim3(1), dim3(OMNI_E), 0, s, *pe, epoch, st, send_base, n_local_rows, need, bucket_cnt, send_cnt,
                             recv_base, limit_ns ? limit_ns : SPIN_LIMIT_NS);
}

cudaError_t omni_launch_ep_barrier(const omni_ep_peers *pe, uint32_t epoch, uint32_t *status, uint64_t limit_ns,
                                   cudaStream_t s) {
    return omni_launch_chain(ep_barrier_kernel, dim3(1), dim3(128), 0, s, *pe, epoch, status, limit_ns);
}

cudaError_t omni_launch_ep_buckets(const int32_t *ids, int T, int world, int32_t *tok_slot, int32_t *bucket_cnt,
                                   int32_t *bucket_list, cudaStream_t s) {
    return omni_launch_chain(ep_bucket_kernel, dim3((T + 255) / 256), dim3(256), 0, s, ids, T, world, tok_slot, bucket_cnt, bucket_list);
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

}  // extern "C"
