// Attention half of a Clef-Omni decoder layer on sm_100a: the step in front of the MoE block.
//   attn_prep_kernel    per-head RMS norm of q and k, interleaved three-axis rotary, q/k/v laid out
//                       per head (reference: metal/clef.metal:2073-2130, omni_attn_prep)
//   attention_kernel    causal grouped-query attention inside each record of the packed batch,
//                       online softmax (reference: metal/clef.metal:2174-2319, omni_attention)
//   dense_tiles_kernel  tile list that lets the expert-product kernel (omni_expert.cu) run the
//                       q|k|v and the output projection as one "expert" over all token rows
//
// attention_kernel: one CTA per (query head, query tile of <= 128 rows of ONE record).  Both
// products run on tcgen05 with operands in 128-byte-swizzled shared memory: S = Q K^T (128 x 128
// keys, accumulator in tensor memory), softmax by 128 threads (one query row each, FP32, running
// maximum and sum), P written back to shared memory as BF16, O_j = P V_j into a second
// accumulator, which the same threads add into their FP32 registers with the usual rescaling.
// Key blocks start at the record's first token, so a token sees the same blocks whether its
// record is packed with others or runs alone.  V is kept transposed ([d][token]) so that both
// products read K-major operands; each record's columns start at a multiple of 64 tokens
// (`vcol`), which keeps every TMA box 16-byte aligned.  Every wait is bounded.
#include <cuda_bf16.h>
#include <type_traits>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "omni_internal.h"
#include "omni_pdl.cuh"
#include "omni_ptx.cuh"

namespace {

constexpr int HD = OMNI_HD, NH = OMNI_NH, NKV = OMNI_NKV;

// ------------------------------------------------------------------ tile list of a dense projection
__global__ void dense_tiles_kernel(int T, omni_ttile *ttiles, int32_t *n_ttiles, int32_t *counters) {
    const int nt = (T + OMNI_TILE_N - 1) / OMNI_TILE_N;
    const int base = T / nt, extra = T % nt;
    for (int j = threadIdx.x; j < nt; j += blockDim.x)
        ttiles[j] = omni_ttile{0, j * base + min(j, extra), base + (j < extra), 0 | (nt << 16)};
    if (threadIdx.x == 0) { *n_ttiles = nt; counters[0] = 0; counters[1] = 0; }
}

// ------------------------------------------------------------------ q/k norm + rotary + layout
// One block per token, four warps, nine heads each (32 query heads, then the 4 key heads).  A lane
// holds four consecutive elements of the 128 of a head (one 8-byte load and store); pair p of a
// head is (element p, element p + 64), so a lane's partners sit in lane ^ 16.  The pair's angle is
// position[axis] * theta^(-p/64) with axis = p % 3 for p < 60 and the temporal axis above (sections
// 24/20/20 interleaved; clef.metal:2051-2053).  The angle is formed and reduced modulo 2 pi in
// FP64 -- FP32 loses ~pos * 6e-8 rad (clef.metal:2055-2060) -- and its cosine and sine, the same
// for every head of the token, are computed once per warp.
__global__ void __launch_bounds__(128) attn_prep_kernel(const __nv_bfloat16 *__restrict__ qkv, const float *__restrict__ qw,
                                                        const float *__restrict__ kw, const int32_t *__restrict__ pos,
                                                        int head_stride, float eps, double theta,
                                                        __nv_bfloat16 *__restrict__ Q, __nv_bfloat16 *__restrict__ K,
                                                        uint32_t *__restrict__ status) {
    dep_wait();
    dep_launch();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long t = blockIdx.x;
    const bool upper = lane >= 16;                                               // elements 64..127: the second of each pair
    // the four pairs of a lane are those of lane ^ 16 too: each computes two and they swap
    float cs[4], sn[4];
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const int own = (upper ? 2 : 0) + j, pair = 4 * (lane & 15) + own, axis = pair < 60 ? pair % 3 : 0;
        const double angle = (double)__ldg(pos + 3 * t + axis) * exp2(-(double)pair * (1.0 / 64.0) * log2(theta));
        const double turns = rint(angle * 0.15915494309189535);
        const float r = (float)fma(-turns, 6.283185307179586, angle);           // |r| <= pi, accurate to FP32 rounding
        float sj, cj;
        sincosf(r, &sj, &cj);
        const float so = __shfl_xor_sync(0xffffffffu, sj, 16), co = __shfl_xor_sync(0xffffffffu, cj, 16);
        cs[own] = cj; sn[own] = sj;
        cs[own ^ 2] = co; sn[own ^ 2] = so;
    }
#pragma unroll
    for (int j = 0; j < 4; j++)
        if (!upper) sn[j] = -sn[j];                                              // lo' = lo cos - hi sin, hi' = hi cos + lo sin
    const float4 wq = __ldg(reinterpret_cast<const float4 *>(qw) + lane), wk = __ldg(reinterpret_cast<const float4 *>(kw) + lane);
    bool bad = false;
    static_assert((NH + NKV) % 4 == 0, "heads are dealt to four warps");
#pragma unroll
    for (int i = 0; i < (NH + NKV) / 4; i++) {            // unrolled: the loads of all nine heads are in flight together
        const int h = warp + 4 * i;
        const bool query = h < NH;
        const uint2 raw = *reinterpret_cast<const uint2 *>(qkv + t * OMNI_QKV + (long)h * HD + 4 * lane);
        float x[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16),
                      __uint_as_float(raw.y & 0xffff0000u)};
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < 4; j++) { bad |= !(fabsf(x[j]) < CUDART_INF_F); sum += x[j] * x[j]; }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
        const float inv = rsqrtf(sum / (float)HD + eps);
        const float4 w = query ? wq : wk;
        x[0] = x[0] * inv * w.x; x[1] = x[1] * inv * w.y; x[2] = x[2] * inv * w.z; x[3] = x[3] * inv * w.w;
        uint32_t o[2];
#pragma unroll
        for (int j = 0; j < 4; j += 2) {
            const float p0 = __shfl_xor_sync(0xffffffffu, x[j], 16), p1 = __shfl_xor_sync(0xffffffffu, x[j + 1], 16);
            const float y0 = x[j] * cs[j] + p0 * sn[j], y1 = x[j + 1] * cs[j + 1] + p1 * sn[j + 1];
            bad |= !(fabsf(y0) < CUDART_INF_F) || !(fabsf(y1) < CUDART_INF_F);
            const __nv_bfloat162 bb = __floats2bfloat162_rn(y0, y1);
            o[j >> 1] = *reinterpret_cast<const uint32_t *>(&bb);
        }
        __nv_bfloat16 *dst = query ? Q + ((long)h * head_stride + t) * HD : K + ((long)(h - NH) * head_stride + t) * HD;
        *reinterpret_cast<uint2 *>(dst + 4 * lane) = make_uint2(o[0], o[1]);
    }
    // reported at completion like the reference's status bit 2 (clef.metal:2120)
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(status, OMNI_ST_ATTN_NONFINITE);
}

// Values, transposed: Vt[kh][d][column of the token].  One block per (64 tokens, key/value head):
// rows read whole (256 bytes per token), written as 64-token runs per head dimension.
__global__ void __launch_bounds__(256) v_transpose_kernel(const __nv_bfloat16 *__restrict__ qkv, const int32_t *__restrict__ vcol,
                                                          int T, int vpitch, __nv_bfloat16 *__restrict__ Vt,
                                                          uint32_t *__restrict__ status) {
    __shared__ unsigned short tile[64][HD + 2];
    __shared__ int col[64];
    dep_wait();
    dep_launch();
    const int t0 = blockIdx.x * 64, kh = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    bool bad = false;
    if (threadIdx.x < 64) col[threadIdx.x] = t0 + threadIdx.x < T ? __ldg(vcol + t0 + threadIdx.x) : -1;
    for (int i = warp; i < 64; i += 8) {
        const long t = t0 + i;
        if (t < T) {
            const uint2 v = *reinterpret_cast<const uint2 *>(qkv + t * OMNI_QKV + (long)(NH + NKV + kh) * HD + lane * 4);
            const unsigned short e[4] = {(unsigned short)(v.x & 0xffff), (unsigned short)(v.x >> 16), (unsigned short)(v.y & 0xffff), (unsigned short)(v.y >> 16)};
#pragma unroll
            for (int k = 0; k < 4; k++) { bad |= (e[k] & 0x7f80) == 0x7f80; tile[i][lane * 4 + k] = e[k]; }
        }
    }
    __syncthreads();
    unsigned short *out = reinterpret_cast<unsigned short *>(Vt) + (long)kh * HD * vpitch;
    for (int d = warp; d < HD; d += 8)
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const int i = lane + 32 * k;
            if (col[i] >= 0) out[(long)d * vpitch + col[i]] = tile[i][d];
        }
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(status, OMNI_ST_ATTN_NONFINITE);
}

// ------------------------------------------------------------------ attention
// One CTA per (pair of query heads that share a key/value head, tile of <= 128 query rows of one
// record).  Key blocks of 128 run from the record's start to the tile's diagonal.  For each head x
// of the pair and block j:
//   S_x(j) = Q_x K_j^T       tcgen05, FP32 in TMEM
//   P_x(j) = exp2(c S - m)   256 threads, two per query row (64 keys each); BF16, two keys per
//                            column, written back over score columns the writing thread alone has
//                            read (keys 0..63 over columns 0..31, keys 64..127 over 96..127)
//   O_x   += P_x(j) V_j      tcgen05 with the A operand read from TMEM, accumulated over all blocks
// The two heads run half a block apart: while one head's threads are in their exponentials the
// tensor pipe forms the other head's value product and next scores, so neither waits for long.
// m is the row's reference maximum.  It follows the running maximum lazily: only when a block's
// maximum exceeds it by more than 2^8 are O and the running sum rescaled (by the softmax threads,
// in TMEM: the scores of a block being there means the previous value product is done);
// otherwise P simply holds values up to 256.  The accumulators never leave TMEM until the end.
struct AttnTile { int32_t rec_start, q0, q_len, vcol0; };          // vcol0: Vt column of the record's first token

constexpr int AT_THREADS = 640;                                    // warp 0 loads, 1 MMA, 2 TMEM, 3 spare, 4..11 softmax of head 0, 12..19 of head 1
constexpr int AT_TILE_BYTES = 128 * 128 * 2;                       // 32 KiB: 128 rows x 128 BF16 as two 64-column halves
constexpr int AT_KV_STAGES = 2;
constexpr int AT_TMEM_COLS = 512;                                  // S_0, S_1, O_0, O_1 of 128 columns each
constexpr int AT_N_BARS = 16;
constexpr int AT_XCH_BYTES = 2 * 2 * 2 * 128 * 4;                  // [head][block parity][row half][row]
constexpr int AT_SMEM_BYTES = AT_TILE_BYTES * (2 + 2 * AT_KV_STAGES) + 1024 + AT_N_BARS * 8 + 64 + AT_XCH_BYTES;
constexpr float AT_LAZY = 8.f;                                     // log2 of how far a block may exceed the reference maximum

__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t *r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(addr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] . B[smem]^T: A's rows are TMEM lanes, two BF16 of the K extent per column.
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {          // 2^x, -inf -> 0; relative error ~2^-22, far below BF16's
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// two FP32 lanes per instruction: (a.x * b.x + c.x, a.y * b.y + c.y) and (a.x + b.x, a.y + b.y)
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(*reinterpret_cast<uint64_t *>(&a)), "l"(*reinterpret_cast<uint64_t *>(&b)),
        "l"(*reinterpret_cast<uint64_t *>(&c)));
    return *reinterpret_cast<float2 *>(&d);
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(*reinterpret_cast<uint64_t *>(&a)), "l"(*reinterpret_cast<uint64_t *>(&b)));
    return *reinterpret_cast<float2 *>(&d);
}

__global__ void __launch_bounds__(AT_THREADS, 1)
attention_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_vt, const AttnTile *__restrict__ tiles, int T, float scale,
                 __nv_bfloat16 *__restrict__ out, uint32_t *__restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *const smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    auto q_smem = [&](int x) { return smem_base + AT_TILE_BYTES * x; };
    auto k_smem = [&](int s) { return smem_base + AT_TILE_BYTES * (2 + s); };
    auto v_smem = [&](int s) { return smem_base + AT_TILE_BYTES * (2 + AT_KV_STAGES + s); };
    const uint32_t bar_base = smem_base + AT_TILE_BYTES * (2 + 2 * AT_KV_STAGES);
    // barriers: q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], o_done[2]
    const uint32_t q_full = bar_base;
    auto k_full = [&](int s) { return bar_base + 8u * (1 + s); };
    auto k_empty = [&](int s) { return bar_base + 8u * (3 + s); };
    auto v_full = [&](int s) { return bar_base + 8u * (5 + s); };
    auto v_empty = [&](int s) { return bar_base + 8u * (7 + s); };
    auto s_full = [&](int x) { return bar_base + 8u * (9 + x); };
    auto p_full = [&](int x) { return bar_base + 8u * (11 + x); };
    auto o_done = [&](int x) { return bar_base + 8u * (13 + x); };
    uint8_t *misc = smem_gen + AT_TILE_BYTES * (2 + 2 * AT_KV_STAGES) + AT_N_BARS * 8;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(misc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(misc + 4);
    volatile int *armed = reinterpret_cast<volatile int *>(misc + 16);         // [5]: q, k stages, v stages (parity of the load in flight, -1 none)
    volatile int *quit = reinterpret_cast<volatile int *>(misc + 40);          // [2] per head: a softmax thread's wait ran out, all of them leave together
    float *xch = reinterpret_cast<float *>(misc + 64);                         // what the two threads of a row tell each other

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const AttnTile tile = tiles[blockIdx.y];                                    // the host lists the tiles with the most key blocks first
    const int h0 = 2 * blockIdx.x, kh = h0 / (NH / NKV);
    const int q_last = tile.q0 + tile.q_len - 1;                                // last query row of the tile
    const int n_blocks = (q_last - tile.rec_start) / 128 + 1;                   // key blocks from the record's start to the diagonal

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; s++) {
            mbar_init(k_full(s), 1); mbar_init(k_empty(s), 1); mbar_init(v_full(s), 1); mbar_init(v_empty(s), 1);
            mbar_init(s_full(s), 1); mbar_init(p_full(s), 256); mbar_init(o_done(s), 1);
        }
        *abort_flag = 0;
        quit[0] = quit[1] = 0;
        for (int i = 0; i < 5; i++) armed[i] = -1;
        fence_mbar_init();
        prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_vt);
    }
    if (warp == 2) { tmem_alloc(smem_u32((const void *)tmem_slot), AT_TMEM_COLS); tmem_relinquish(); }
    dep_wait();
    dep_launch();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------- loads: both Q tiles once, then K one block ahead of Vt
        armed[0] = 0;
        mbar_expect_tx(q_full, 2 * AT_TILE_BYTES);
        for (int x = 0; x < 2; x++) {
            tma_load_2d(q_smem(x), &tm_q, 0, (h0 + x) * T + tile.q0, q_full);                        // d 0..63
            tma_load_2d(q_smem(x) + AT_TILE_BYTES / 2, &tm_q, 64, (h0 + x) * T + tile.q0, q_full);   // d 64..127
        }
        PipeState pk, pv;
        auto load_k = [&](int j) {
            if (!mbar_wait(k_empty(pk.stage), pk.phase ^ 1u, abort_flag, status)) return false;
            const int key0 = tile.rec_start + j * 128;
            armed[1 + pk.stage] = (int)pk.phase;
            mbar_expect_tx(k_full(pk.stage), AT_TILE_BYTES);
            tma_load_2d(k_smem(pk.stage), &tm_k, 0, kh * T + key0, k_full(pk.stage));
            tma_load_2d(k_smem(pk.stage) + AT_TILE_BYTES / 2, &tm_k, 64, kh * T + key0, k_full(pk.stage));
            pk.advance(AT_KV_STAGES);
            return true;
        };
        bool ok = load_k(0);
        for (int j = 0; j < n_blocks && ok; j++) {
            if (j + 1 < n_blocks) ok = load_k(j + 1);
            if (!ok || !mbar_wait(v_empty(pv.stage), pv.phase ^ 1u, abort_flag, status)) break;
            armed[3 + pv.stage] = (int)pv.phase;
            mbar_expect_tx(v_full(pv.stage), AT_TILE_BYTES);
            tma_load_2d(v_smem(pv.stage), &tm_vt, tile.vcol0 + j * 128, kh * HD, v_full(pv.stage));            // keys 0..63 of the block
            tma_load_2d(v_smem(pv.stage) + AT_TILE_BYTES / 2, &tm_vt, tile.vcol0 + j * 128 + 64, kh * HD, v_full(pv.stage));
            pv.advance(AT_KV_STAGES);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------------------------------------------------- MMA issuer
        // Per head and block: the value product as soon as P is written, and behind it the head's next
        // scores into the same TMEM columns (the tensor pipe runs them in the order issued, so the
        // product has read P before the scores overwrite it).
        const uint32_t idesc = idesc_bf16(128, 128);
        auto scores = [&](int x, int stage) {     // S_x = Q_x K^T over the 128 head dimensions: two 64-wide halves, four K=16 steps each
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const uint64_t da = smem_desc_sw128(q_smem(x) + half * (AT_TILE_BYTES / 2));
                const uint64_t db = smem_desc_sw128(k_smem(stage) + half * (AT_TILE_BYTES / 2));
#pragma unroll
                for (int k = 0; k < 4; k++) umma_bf16(tmem_base + x * 128, da + 2u * k, db + 2u * k, idesc, (half | k) ? 1u : 0u);
            }
            umma_commit(s_full(x));
        };
        PipeState pk, pv;
        bool ok = mbar_wait(q_full, 0, abort_flag, status) && mbar_wait(k_full(0), 0, abort_flag, status);
        if (ok) {
            tc_fence_after();
            scores(0, 0); scores(1, 0);
            umma_commit(k_empty(0));
            pk.advance(AT_KV_STAGES);
        }
        for (int j = 0; j < n_blocks && ok; j++) {
            for (int x = 0; x < 2 && ok; x++) {
                ok = mbar_wait(p_full(x), (uint32_t)j & 1u, abort_flag, status);
                if (ok && x == 0) ok = mbar_wait(v_full(pv.stage), pv.phase, abort_flag, status);
                if (!ok) break;
                tc_fence_after();
                // O_x += P_x V: the 128 keys of the block are eight K=16 steps, 8 TMEM columns of P each
                // (keys 0..63 in columns 0..31 of the score buffer, keys 64..127 in columns 96..127)
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const uint64_t db = smem_desc_sw128(v_smem(pv.stage) + (k >> 2) * (AT_TILE_BYTES / 2));
                    umma_bf16_ts(tmem_base + 256 + x * 128, tmem_base + x * 128 + 8 * k + (k >> 2) * 64, db + 2u * (k & 3), idesc, (j | k) ? 1u : 0u);
                }
                if (x == 1) umma_commit(v_empty(pv.stage));
                if (j + 1 < n_blocks) {
                    if (x == 0) { ok = mbar_wait(k_full(pk.stage), pk.phase, abort_flag, status); if (!ok) break; tc_fence_after(); }
                    scores(x, pk.stage);
                    if (x == 1) umma_commit(k_empty(pk.stage));
                } else {
                    umma_commit(o_done(x));
                }
            }
            pv.advance(AT_KV_STAGES);
            pk.advance(AT_KV_STAGES);
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------- softmax of one head: two threads per query row
        // Thread (row r, half hf) owns keys hf*64.. of every score block, the P columns that hold
        // them, and head dimensions hf*64.. of the accumulator.  The two threads of a row sit in
        // different warps and exchange their partial maxima through shared memory at the head's
        // named barrier; a thread whose wait ran out marks `quit` and still joins that barrier,
        // after which all threads of the head leave together.
        const int x = (warp - 4) >> 3, q4 = warp & 3, hf = ((warp - 4) >> 2) & 1;
        const int r = q4 * 32 + lane;                                             // row inside the tile = TMEM lane
        const uint32_t tmem_s = tmem_base + x * 128 + ((uint32_t)(q4 * 32) << 16);
        const uint32_t tmem_o = tmem_base + 256 + x * 128 + ((uint32_t)(q4 * 32) << 16) + hf * 64;
        float *xc = xch + x * 512;                                                // [parity][half][row]
        const float c = scale * 1.4426950408889634f;                              // scores to log2 units
        float m = 0.f, l = 0.f;
        bool alive = true;
        for (int j = 0; j < n_blocks; j++) {
            const int par = j & 1;
            if (alive) alive = mbar_wait(s_full(x), (uint32_t)par, abort_flag, status);
            alive = __all_sync(0xffffffffu, alive);
            const bool diagonal = j == n_blocks - 1;                              // the only block with keys after some of the rows
            uint32_t ta[32];
            float pmax = -CUDART_INF_F;
            if (alive) {
                tc_fence_after();
                // two sweeps over the thread's 64 scores, 32 at a time: the maximum first, then the
                // probabilities (reading TMEM twice costs less than holding the scores in registers)
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    tmem_ld32(tmem_s + hf * 64 + q * 32, ta);
                    tmem_ld_wait();
                    if (diagonal) {
#pragma unroll
                        for (int i = 0; i < 32; i++)
                            if (hf * 64 + q * 32 + i > r) ta[i] = 0xff800000u;
                    }
                    float mq = fmaxf(__uint_as_float(ta[0]), __uint_as_float(ta[1]));
#pragma unroll
                    for (int i = 2; i < 32; i += 2) mq = max3(mq, __uint_as_float(ta[i]), __uint_as_float(ta[i + 1]));
                    pmax = fmaxf(pmax, mq);
                }
                xc[(par * 2 + hf) * 128 + r] = pmax;
            } else {
                quit[x] = 1;
            }
            asm volatile("bar.sync %0, 256;" ::"r"(1 + x) : "memory");
            if (quit[x]) { alive = false; break; }
            // key 0 of every block is visible to every row (tiles and blocks are both cut from the
            // record's start in steps of 128), so the block maximum is finite
            const float bm = fmaxf(pmax, xc[(par * 2 + (hf ^ 1)) * 128 + r]) * c;
            float corr = 1.f;
            if (j == 0) m = bm;
            else if (bm > m + AT_LAZY) { corr = ex2_approx(m - bm); m = bm; l *= corr; }
            if (__any_sync(0xffffffffu, corr != 1.f)) {
                // the scores of this block being complete means the previous value product is: O is at rest
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    uint32_t t32[32];
                    tmem_ld32(tmem_o + q * 32, t32);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++) t32[i] = __float_as_uint(__uint_as_float(t32[i]) * corr);
                    tmem_st32(tmem_o + q * 32, t32);
                }
            }
            // P = exp2(c s - m) as BF16 (values up to 2^8 while m lags the running maximum), two keys per column
            uint32_t pk[32];
            float2 acc[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
            const float2 c2 = make_float2(c, c), nm2 = make_float2(-m, -m);
#pragma unroll
            for (int q = 0; q < 2; q++) {
                tmem_ld32(tmem_s + hf * 64 + q * 32, ta);
                tmem_ld_wait();
                if (diagonal) {
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        if (hf * 64 + q * 32 + i > r) ta[i] = 0xff800000u;
                }
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const float2 e = ffma2(make_float2(__uint_as_float(ta[2 * i]), __uint_as_float(ta[2 * i + 1])), c2, nm2);
                    const float2 pp = make_float2(ex2_approx(e.x), ex2_approx(e.y));
                    acc[i & 1] = fadd2(acc[i & 1], pp);
                    const __nv_bfloat162 bb = __floats2bfloat162_rn(pp.x, pp.y);
                    pk[q * 16 + i] = *reinterpret_cast<const uint32_t *>(&bb);
                }
            }
            l += (acc[0].x + acc[1].x) + (acc[0].y + acc[1].y);
            // P goes over columns whose scores this thread alone read: keys 0..63 into columns 0..31,
            // keys 64..127 into columns 96..127
            tmem_st32(tmem_s + hf * 96, pk);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(p_full(x));
        }
        // the row's denominator is the sum of what its two threads added up (same reference maximum in both)
        if (alive) alive = mbar_wait(o_done(x), 0, abort_flag, status);
        alive = __all_sync(0xffffffffu, alive);
        if (!alive) quit[x] = 1;
        xc[((n_blocks & 1) * 2 + hf) * 128 + r] = l;
        asm volatile("bar.sync %0, 256;" ::"r"(1 + x) : "memory");
        if (!quit[x]) {
            tc_fence_after();
            const float lt = l + xc[((n_blocks & 1) * 2 + (hf ^ 1)) * 128 + r];
            const float inv = lt > 0.f ? 1.f / lt : 0.f;
            const int qg = tile.q0 + r;                                           // global token index of the row
            uint4 *dst = reinterpret_cast<uint4 *>(out + (long)qg * (NH * HD) + (h0 + x) * HD + hf * 64);
#pragma unroll
            for (int q = 0; q < 2; q++) {
                uint32_t t32[32];
                tmem_ld32(tmem_o + q * 32, t32);
                tmem_ld_wait();
                if (r < tile.q_len) {
#pragma unroll
                    for (int ch = 0; ch < 4; ch++) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const __nv_bfloat162 bb = __floats2bfloat162_rn(__uint_as_float(t32[ch * 8 + 2 * i]) * inv,
                                                                            __uint_as_float(t32[ch * 8 + 2 * i + 1]) * inv);
                            w[i] = *reinterpret_cast<const uint32_t *>(&bb);
                        }
                        dst[q * 4 + ch] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        // a wait ran out: give loads already in flight a bounded chance to land
        for (int s = 0; s < 5; s++) {
            const int par = armed[s];
            if (par < 0) continue;
            const uint32_t bar = s == 0 ? q_full : s < 3 ? k_full(s - 1) : v_full(s - 3);
            const uint64_t t0 = globaltimer_ns();
            while (!mbar_try_wait(bar, (uint32_t)par) && globaltimer_ns() - t0 < 50000000ull) {}
        }
    }
    __syncthreads();
    if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem_base, AT_TMEM_COLS); }
}

}  // namespace

extern "C" {


cudaError_t omni_attn_configure(void) {
    return cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM_BYTES);
}

cudaError_t omni_launch_dense_tiles(int T, omni_ttile *ttiles, int32_t *n_ttiles, int32_t *counters, cudaStream_t s) {
    dense_tiles_kernel<<<1, 128, 0, s>>>(T, ttiles, n_ttiles, counters);
    return cudaGetLastError();
}

cudaError_t omni_launch_attn_prep(const void *qkv, const float *qw, const float *kw, const int32_t *pos, const int32_t *vcol, int T,
                                  int head_stride, int vpitch, float eps, double theta, void *Q, void *K, void *Vt, uint32_t *status,
                                  cudaStream_t s) {
    cudaError_t e = omni_launch_chain(attn_prep_kernel, dim3(T), dim3(128), 0, s, (const __nv_bfloat16 *)qkv, qw, kw, pos, head_stride, eps,
                                      theta, (__nv_bfloat16 *)Q, (__nv_bfloat16 *)K, status);
    if (e != cudaSuccess) return e;
    return omni_launch_chain(v_transpose_kernel, dim3((T + 63) / 64, OMNI_NKV), dim3(256), 0, s, (const __nv_bfloat16 *)qkv, vcol, T, vpitch,
                             (__nv_bfloat16 *)Vt, status);
}

// tiles: [n_tiles] of {record start, first query row, rows (<= 128), Vt column of the record start}
cudaError_t omni_launch_attention(const CUtensorMap *tm_q, const CUtensorMap *tm_k, const CUtensorMap *tm_vt, const void *tiles,
                                  int n_tiles, int T, void *out, uint32_t *status, cudaStream_t s) {
    return omni_launch_chain(attention_kernel, dim3(OMNI_NH / 2, n_tiles), dim3(AT_THREADS), AT_SMEM_BYTES, s, *tm_q, *tm_k, *tm_vt,
                             (const AttnTile *)tiles, T, 1.0f / sqrtf((float)OMNI_HD), (__nv_bfloat16 *)out, status);
}

}  // extern "C"
