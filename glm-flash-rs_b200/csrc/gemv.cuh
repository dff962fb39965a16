// Grouped EXL3 GEMV for windows of 1..16 rows (decode and speculative verify), sm_100a.
//
// Replaces upstream's exl3_grouped_8_4 / exl3_load_nc_8_1 + gateup_epilogue_kernel + down_epilogue_kernel
// (native/exl3.cu:59-170,260-321, native/expert_loads.cu:130-285).  Same operands and the same member /
// pair conventions; a different machine mapping:
//
//   * work item = (distinct expert u, 128-column block nb, K split): MATS matrices x KTC k-tiles x 8 n-tiles,
//     i.e. MATS x KTC contiguous 1-KB rows of packed trellis words.  They are all requested as TMA bulk copies
//     (cp.async.bulk) into shared memory at kernel start, four k-tiles per mbarrier, so the whole item is in flight
//     before anything else happens and the copy engine, not the warps, follows the stream.
//   * a lane reads 16 bytes (4 words of one tile) with one LDS.128: that is 32 weights, all 16 k of two
//     columns (G, G+8), so only one shuffle per 32 weights is needed for the word that precedes the chunk.
//     The four lanes of a quad read the same 16-byte slot of four consecutive k-tiles.
//   * states are cut with funnel shifts in pairs (state_j << 16 | state_{j+4}), multiplied by the codebook
//     constant, masked, and the two fp16 halves of a codeword are added by one HADD2 whose result carries the
//     weight in both halves: exactly upstream's fp16 weight (bit-exact decode), without byte permutes.
//   * the weights are the A operand of mma.m16n8k16 (rows = 16 output columns) over a doubled K: the pair
//     (w, w) meets (x_k, 0), so a.w is accumulated once, in fp32.  Members (<= 8 per set) are the N dimension;
//     a second set of B operands serves experts with 9..16 members without decoding twice.
//   * warps of a CTA own disjoint n-tiles (and matrices), so nothing is reduced across warps;
//     the K splits of an (expert, column block) are the CTAs of one thread-block cluster: each leaves its
//     fp32 partial in its own shared memory, and after a cluster barrier the members are finished by the CTAs
//     round robin, reading the peers' partials through distributed shared memory and adding them in ascending
//     split order before the epilogue: Hadamard, scales, SwiGLU, down-input rotation (MATS = 2) or Hadamard and
//     output scale (MATS = 1).  No global scratch, no atomics, no value depends on arrival order.
//   * every pair's result depends only on its own row: the split count and tiling are fixed by the shape, and
//     mma keeps columns (members) independent, so a row of a 16-row window has the bits of the 1-row call.
#pragma once
#include "common.cuh"

namespace gf {

// GF_PROBE (timing experiments only, wrong results, in the spirit of upstream's PROBE modes,
// native/expert_loads.cu:46-47): 1 = no decode / mma, 2 = no partial exchange and epilogue, 3 = both.
#ifndef GF_PROBE
#define GF_PROBE 0
#endif
// GF_TRACE (timing experiments only): thread 0 of every CTA stamps the global nanosecond timer at the phase boundaries
// into a buffer registered with glmflash_trace_set(): [MATS - 1][(u * splits + split) * 16 + nb (< 16384)][16] int64.
#ifdef GF_TRACE
static __device__ long long *g_trace = nullptr;    // one copy per translation unit; experts.cu owns the used one
#define GF_STAMP(i)                                                                                              \
    do {                                                                                                         \
        if (threadIdx.x == 0 && g_trace) {                                                                       \
            long long t_;                                                                                        \
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_));                                                \
            g_trace[(((size_t)(MATS - 1) * 16384 + ((size_t)(u * gridDim.y + split) * 16 + nb)) << 4) + (i)] = t_; \
        }                                                                                                        \
    } while (0)
#define GF_STAMP_SMID(i)                                                                                         \
    do {                                                                                                         \
        if (threadIdx.x == 0 && g_trace) {                                                                       \
            unsigned t_;                                                                                         \
            asm volatile("mov.u32 %0, %smid;" : "=r"(t_));                                                       \
            g_trace[(((size_t)(MATS - 1) * 16384 + ((size_t)(u * gridDim.y + split) * 16 + nb)) << 4) + (i)] = t_; \
        }                                                                                                        \
    } while (0)
#else
#define GF_STAMP(i) do { } while (0)
#define GF_STAMP_SMID(i) do { } while (0)
#endif
constexpr int GEMV_THREADS = 256;
constexpr int GEMV_MAX_SPLITS = 8;                 // K splits of an item = CTAs of a cluster (portable maximum)
constexpr int GEMV_WROW = 1024 + 32;               // bytes per staged weight row (1 KB + 32 B: conflict-free LDS.128)
constexpr int GEMV_PST = 132;                      // floats per partial row

enum GemvMode : int { GEMV_GATEUP = 0, GEMV_DOWN = 1, GEMV_LINEAR = 2 };

// Barrier of one warp pair (64 threads); ids 1..4, compile-time so that only five barriers are reserved per CTA.
__device__ __forceinline__ void pair_barrier(int pw) {
    switch (pw) {
        case 0: asm volatile("bar.sync 1, 64;" ::: "memory"); break;
        case 1: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
        case 2: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
        default: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
    }
}

struct GemvArgs {
    const __half *X0, *X1;        // rotated inputs [P][K] fp16 (X1: second matrix, MATS = 2)
    const uint32_t *T0, *T1;      // trellis banks [E1][K/16][N/16][32]
    const int *ids, *count, *members;
    const __half *sv0, *sv1, *sd; // gate/up: svh_g, svh_u, suh_d;  down / linear: svh_d
    __half *xd;                   // gate/up out: [P][N] fp16;  linear out: [P][N] fp16
    float *y;                     // down out: [P][N] fp32
    int *status;
    int K, N, P, SK, KTC, maxm, slots, E, e_lo, e_hi, shared_exl3, mode;
    float limit;
    // fused front end (the layer pipeline of windows of <= 16 rows): with picks != nullptr the CTA derives its expert
    // and members from the routing table itself (no grouping kernel), with xin != nullptr it rotates the layer input
    // itself (no rotation kernel, no Xg / Xu round trip).  wait_first: picks / xin may be the previous kernel's output.
    const int *picks;
    const __nv_bfloat16 *xin;
    const __half *suh0, *suh1;
    int rows, x_stride, wait_first;
};

// Position of the n-th (0-based) set bit of w (which has more than n set bits): five popcount steps.
__device__ __forceinline__ int nth_set_bit(uint32_t w, int n) {
    int pos = 0;
#pragma unroll
    for (int width = 16; width >= 1; width >>= 1) {
        const int c = __popc(w & ((1u << width) - 1u));
        if (n >= c) { n -= c; w >>= width; pos += width; }
    }
    return pos;
}

__device__ __forceinline__ bool expert_skipped(int e, int E, int shared_exl3, int e_lo, int e_hi) {
    // the window [e_lo, e_hi) selects routed experts; the shared expert (id E) is governed by shared_exl3 alone
    return e < 0 || e > E || (e == E ? !shared_exl3 : (e < e_lo || e >= e_hi));
}

// (w, w) from a masked codeword: one half-precision add of its two halves.
__device__ __forceinline__ uint32_t weight_dup(uint32_t x) {
    const __half2 v = *reinterpret_cast<const __half2 *>(&x);
    const __half2 r = __hadd2(__low2half2(v), __high2half2(v));
    return *reinterpret_cast<const uint32_t *>(&r);
}

// K split of a shape: k-tiles per CTA and the number of splits (<= 8, the cluster size); sk * ktc == K / 16 always.
// Powers of two times 16 k-tiles where that divides K / 16 (2048: 8 x 16, 1536: 6 x 16, 4096: 8 x 32); other multiples
// of 256 take the largest split count whose share is a whole number of 128-k Hadamard blocks (2304: 6 x 24).
inline void gemv_split(int K, int &ktc, int &sk) {
    const int KT = K / 16;
    ktc = 16;
    while (KT / ktc > GEMV_MAX_SPLITS) ktc *= 2;
    sk = KT / ktc;
    if (sk * ktc == KT) return;
    for (sk = GEMV_MAX_SPLITS; sk > 1; --sk)
        if (KT % sk == 0 && (KT / sk) % 8 == 0) break;
    ktc = KT / sk;
}
// dynamic shared memory size of a launch
inline size_t gemv_smem_bytes(int mats, int sets, int ktc) {
    size_t w = (size_t)mats * ktc * GEMV_WROW;
    size_t part = (size_t)mats * sets * 8 * GEMV_PST * sizeof(float);
    size_t a = sets == 2 ? (size_t)mats * sets * 8 * (ktc * 8 + 4) * 4 : (size_t)mats * sets * 8 * (ktc * 16 + 8) * 4;
    return 128 + (w > part ? w : part) + a;
}

// Work item (cluster) = (distinct expert u, 128-column block nb); CTA `split` of the cluster owns K split `split`:
// MATS x KTC rows of 1 KB.  8 warps.  MATS = 2: warp = (matrix, pair of n-tiles).  MATS = 1: warp = n-tile.
// Returns 0 after a computed item, 1 when u is beyond the distinct experts of the window, 2 when the expert is outside
// this rank's window.
template <int MATS, int SETS>
__device__ __forceinline__ int gemv_item(const GemvArgs &a, unsigned char *smem, const int nb, const int split, const int u) {
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);                         // one barrier per 4 k-tiles (<= 16)
    unsigned char *wsm = smem + 128;                                             // [MATS][KTC] rows of GEMV_WROW
    constexpr bool PACKED = SETS == 2;               // layout of the staged activations, see below
    const int KTC = a.KTC, NG = KTC >> 2, KC = KTC * 16, AST = PACKED ? (KC >> 1) + 4 : KC + 8;   // dwords per member row
    const size_t wbytes = (size_t)MATS * KTC * GEMV_WROW;
    constexpr size_t PBYTES = (size_t)MATS * SETS * 8 * GEMV_PST * sizeof(float);
    const size_t wp = wbytes > PBYTES ? wbytes : PBYTES;
    float *part = reinterpret_cast<float *>(wsm);                                // aliases wsm after the K loop
    uint32_t *asm_ = reinterpret_cast<uint32_t *>(wsm + wp);                     // [MATS][SETS*8][AST]
    __shared__ int rows_sh[16];
    __shared__ float scale_sh[3][128];                                           // epilogue scale vectors of (e, nb)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = lane >> 2, T = lane & 3;
    const int KT = a.K >> 4, NTILES = a.N >> 4;

    GF_STAMP(0);
    if (tid == 0) {
        for (int g = 0; g < NG; ++g) {
            mbar_init(bars + g, 1);
            mbar_expect_tx(bars + g, MATS * 4 * 1024);   // the one arrival; the copies below complete the byte count
        }
        mbar_fence_init();
    }
    if (a.wait_first) pdl_wait();                   // the routing table / layer input may belong to the kernel before
    GF_STAMP_SMID(13);
    int cnt = 0, e = -1;
    if (a.picks && a.rows == 1) {
        // ---- one row: the distinct experts are the row's picks in ascending order; every warp finds number u itself
        //      (one load, a few shuffles, no block barrier).  A pick that repeats an earlier slot does not count.
        //      Only experts this GPU computes count (expert window, shared-expert switch), so that the launch needs no
        //      more clusters than the window has experts.
        constexpr int NONE = 0x7fffffff;
        int pk = lane < a.slots ? __ldcg(a.picks + lane) : NONE;
        int sh = a.shared_exl3;
        if (sh == 2) {
            // the shared expert goes to the rank with the fewest distinct routed picks of the row (shared_owner_rank's rule,
            // evaluated on the row's picks held by the lanes)
            const int W = a.e_hi - a.e_lo, ranks = (a.E + W - 1) / W;
            int c = 0;
            for (int j = 0; j < a.slots; ++j) {
                const int v = __shfl_sync(0xffffffffu, pk, j);
                bool vdup = false;
                for (int q = 0; q < j; ++q) vdup |= __shfl_sync(0xffffffffu, pk, q) == v;
                if (!vdup && v >= 0 && v < a.E && v / W == lane) c++;
            }
            int best = (lane < ranks ? c : 1023) * 32 + lane;
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, d));
            sh = (best & 31) == a.e_lo / W;
        }
        if (pk != NONE && expert_skipped(pk, a.E, sh, a.e_lo, a.e_hi)) pk = NONE;
        bool dup = false;
        int rank_lt = 0, distinct = 0;
        for (int j = 0; j < a.slots; ++j) {
            const int v = __shfl_sync(0xffffffffu, pk, j);
            bool vdup = v == NONE;
            for (int q = 0; q < j; ++q) vdup |= __shfl_sync(0xffffffffu, pk, q) == v;
            if (j < lane && v == pk) dup = true;
            if (!vdup) { distinct++; if (v < pk) rank_lt++; }
        }
        const uint32_t hit = __ballot_sync(0xffffffffu, pk != NONE && !dup && rank_lt == u);
        GF_STAMP(14);
        cnt = distinct;
        const int slot = hit ? __ffs(hit) - 1 : 0;
        e = hit ? __shfl_sync(0xffffffffu, pk, slot) : -1;
        if (u >= cnt) return 1;                                // uniform for the whole cluster
        if (expert_skipped(e, a.E, a.shared_exl3, a.e_lo, a.e_hi)) return 2;
        if (tid < 16) rows_sh[tid] = tid == 0 ? slot : -1;
    } else if (a.picks) {
        // ---- grouping in the CTA: distinct expert number u of the window and its members, from the routing table
        __shared__ uint32_t used_sh[32];
        if (tid < 32) used_sh[tid] = 0u;
        __syncthreads();
        const int np = a.rows * a.slots;
        for (int i = tid; i < np; i += GEMV_THREADS) {
            const int pk = __ldcg(a.picks + i);
            if (pk >= 0 && pk <= a.E) atomicOr(&used_sh[pk >> 5], 1u << (pk & 31));   // ids above E name nothing
        }
        __syncthreads();
        __shared__ int e_sh, cnt_sh;
        if (warp == 0) {                                       // number u among the set bits: one bitmap word per lane
            // experts another GPU computes do not count (see the one-row form): the expert window, and the shared expert
            // by the config's switch or, when its owner is decided per window, by shared_owner_rank
            int sh = a.shared_exl3;
            if (sh == 2) sh = shared_owner_rank(used_sh, a.E, a.e_hi - a.e_lo, lane) == a.e_lo / (a.e_hi - a.e_lo);
            const int lo = min(max(a.e_lo - 32 * lane, 0), 32), hi = min(max(a.e_hi - 32 * lane, 0), 32);
            uint32_t keep = hi > lo ? ((hi == 32 ? 0xffffffffu : (1u << hi) - 1u) & ~((1u << lo) - 1u)) : 0u;
            if (sh && (a.E >> 5) == lane) keep |= 1u << (a.E & 31);
            const uint32_t bts = used_sh[lane] & keep;
            const int c = __popc(bts);
            int incl = c;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += up;
            }
            const int excl = incl - c;
            if (lane == 31) cnt_sh = incl;
            if (u >= excl && u < incl) e_sh = lane * 32 + nth_set_bit(bts, u - excl);
            if (lane == 31 && u >= incl) e_sh = -1;
        }
        __syncthreads();
        e = e_sh; cnt = cnt_sh;
        if (u >= cnt) return 1;                                // uniform for the whole cluster
        if (expert_skipped(e, a.E, a.shared_exl3, a.e_lo, a.e_hi)) return 2;
        if (warp == 0) {                                       // rows <= 16: one lane per row, ascending row order
            int slot = -1;
            if (lane < a.rows)
                for (int sl = a.slots - 1; sl >= 0; --sl)
                    if (__ldcg(a.picks + lane * a.slots + sl) == e) slot = sl;
            const uint32_t ball = __ballot_sync(0xffffffffu, slot >= 0);
            const int pos = __popc(ball & ((1u << lane) - 1u));
            if (slot >= 0 && pos < 16) rows_sh[pos] = lane * a.slots + slot;
            if (lane < 16 && lane >= __popc(ball)) rows_sh[lane] = -1;
        }
    } else {
        // one round trip for everything the prologue needs (none of the three loads depends on another)
        cnt = __ldcg(a.count);
        e = __ldcg(a.ids + u);
        int code = -1;
        if (tid < 16 && tid < a.maxm) code = __ldcg(a.members + (size_t)u * a.maxm + tid);
        if (u >= cnt) return 1;                                // uniform for the whole cluster
        if (expert_skipped(e, a.E, a.shared_exl3, a.e_lo, a.e_hi)) return 2;
        if (tid < 16) rows_sh[tid] = code >= 0 ? (code >> 5) * a.slots + (code & 31) : -1;
    }
    GF_STAMP(15);
    __syncthreads();
    GF_STAMP(1);

    int nmem = 0;
#pragma unroll
    for (int m = 0; m < SETS * 8; ++m) nmem += rows_sh[m] >= 0;   // members come first
    const int kt0 = split * KTC, k0 = kt0 * 16;

    // ---- small operands first: the scale vectors of (e, nb) and the first rotation item of every warp are requested
    //      BEFORE the weight stream, so that they do not queue behind it in the memory system
    unsigned short sc0 = 0, sc1 = 0, sc2 = 0;      // raw fp16 bits; converted where they are stored, after the rotation
    if (tid < 128) {                               // constants of the bank: no dependency on the kernel before
        const size_t o = (size_t)e * a.N + nb * 128 + tid;
        sc0 = __ldg(reinterpret_cast<const unsigned short *>(a.sv0) + o);
        if (MATS == 2) {
            sc1 = __ldg(reinterpret_cast<const unsigned short *>(a.sv1) + o);
            sc2 = __ldg(reinterpret_cast<const unsigned short *>(a.sd) + o);
        }
    }
    // rotation items (xin path): one warp per (matrix, member, 128-block of this K range)
    const int blocks = KC >> 7;
    const int rot_items = a.xin ? MATS * nmem * blocks : 0;
    uint2 rot_x = make_uint2(0u, 0u), rot_s = make_uint2(0u, 0u);
    auto rot_load = [&](int it) {
        const int blk = it % blocks, mm = it / blocks;
        const int m = mm % nmem, mat = mm / nmem;
        const int row = rows_sh[m] / a.slots;
        const int kl = blk * 128 + 4 * lane;
        rot_x = __ldcg(reinterpret_cast<const uint2 *>(a.xin + (size_t)row * a.x_stride + k0 + kl));
        rot_s = __ldg(reinterpret_cast<const uint2 *>((mat ? a.suh1 : a.suh0) + (size_t)e * a.K + k0 + kl));
    };
    const bool rot_early = a.wait_first != 0 && warp < rot_items;   // x is complete only after the dependency wait
    if (rot_early) rot_load(warp);

    // ---- the whole item's packed words, in flight at once, the requests spread over the warps (an issuing thread is
    //      held while the copy engine accepts its request)
    {
        constexpr int WARPS = GEMV_THREADS / 32;
        const int per_warp = (MATS * KTC + WARPS - 1) / WARPS;
        const int r = warp * per_warp + lane;
        if (lane < per_warp && r < MATS * KTC) {
            const int mat = r / KTC, ktl = r % KTC;
            const uint32_t *T_ = mat ? a.T1 : a.T0;
            const uint32_t *src = T_ + (((size_t)e * KT + kt0 + ktl) * NTILES + (size_t)nb * 8) * 32;
            tma_load_1d(wsm + (size_t)r * GEMV_WROW, src, 1024, bars + (ktl >> 2));
        }
    }
    pdl_launch_dependents();
    GF_STAMP(2);
    bool ok = true;
    pdl_wait();                                   // X belongs to the kernel before this one (no-op after wait_first)
    GF_STAMP(3);

    // ---- stage the members' activations of this K range, one row of AST dwords per member.
    //      PACKED (two member sets): fp16, natural k order (AST = KC / 2 + 4 keeps the 16-byte reads of the K loop free
    //      of bank conflicts); the (x_k, 0) operand pairs are cut in the K loop.  This halves the staging area, which is
    //      what lets four CTAs share an SM.
    //      Otherwise (one set): ready-made (x_k, 0) dword pairs, permuted to the mma order: the pair of local
    //      k = 64 g + 16 T + 8 h + 2 t + b sits at dword g*64 + (2t + h)*8 + 2T + b.
    auto stage_pos = [](int kl) {
        const int g = kl >> 6, TT = (kl >> 4) & 3, h = (kl >> 3) & 1, t = (kl >> 1) & 3;
        return g * 64 + (2 * t + h) * 8 + 2 * TT;
    };
    //      Rows of absent members are left as they are: an mma column depends on its own B column only, and the
    //      columns of absent members are never stored.
    if (a.xin) {
        // rotate the layer input here (upstream rot_in_kernel, native/exl3.cu:224-241):
        // fp16(H(x * suh) / sqrt 128), the same butterflies and rounding as the kernel form
        for (int it = warp; it < rot_items; it += GEMV_THREADS / 32) {
            if (!(rot_early && it == warp)) rot_load(it);
            const int blk = it % blocks, mm = it / blocks;
            const int m = mm % nmem, mat = mm / nmem;
            const int kl = blk * 128 + 4 * lane;
            const __nv_bfloat162 x01 = *reinterpret_cast<const __nv_bfloat162 *>(&rot_x.x),
                                 x23 = *reinterpret_cast<const __nv_bfloat162 *>(&rot_x.y);
            const __half2 s01 = *reinterpret_cast<const __half2 *>(&rot_s.x), s23 = *reinterpret_cast<const __half2 *>(&rot_s.y);
            float v[4] = {__bfloat162float(x01.x) * __low2float(s01), __bfloat162float(x01.y) * __high2float(s01),
                          __bfloat162float(x23.x) * __low2float(s23), __bfloat162float(x23.y) * __high2float(s23)};
            fwht128(v, lane);
            const __half2 r01 = __halves2half2(__float2half_rn(v[0] * HAD_SCALE), __float2half_rn(v[1] * HAD_SCALE));
            const __half2 r23 = __halves2half2(__float2half_rn(v[2] * HAD_SCALE), __float2half_rn(v[3] * HAD_SCALE));
            const uint32_t w01 = *reinterpret_cast<const uint32_t *>(&r01), w23 = *reinterpret_cast<const uint32_t *>(&r23);
            uint32_t *dst = asm_ + ((size_t)mat * SETS * 8 + m) * AST;
            if (PACKED) {
                *reinterpret_cast<uint2 *>(dst + (kl >> 1)) = make_uint2(w01, w23);
            } else {
                *reinterpret_cast<uint2 *>(dst + stage_pos(kl)) = make_uint2(w01 & 0xffffu, w01 >> 16);
                *reinterpret_cast<uint2 *>(dst + stage_pos(kl + 2)) = make_uint2(w23 & 0xffffu, w23 >> 16);
            }
        }
    } else {
        const int half = KC >> 1;
        const int items = MATS * nmem * half;
        for (int i = tid; i < items; i += GEMV_THREADS) {
            const int kp = i % half, mm = i / half;
            const int m = mm % nmem, mat = mm / nmem;
            const int p = rows_sh[m];
            const uint32_t v = __ldcg(reinterpret_cast<const uint32_t *>((mat ? a.X1 : a.X0) + (size_t)p * a.K + k0) + kp);
            uint32_t *dst = asm_ + ((size_t)mat * SETS * 8 + m) * AST;
            if (PACKED) dst[kp] = v;
            else *reinterpret_cast<uint2 *>(dst + stage_pos(2 * kp)) = make_uint2(v & 0xffffu, v >> 16);
        }
    }
    if (tid < 128) {
        scale_sh[0][tid] = __half2float(__ushort_as_half(sc0));
        if (MATS == 2) {
            scale_sh[1][tid] = __half2float(__ushort_as_half(sc1));
            scale_sh[2][tid] = __half2float(__ushort_as_half(sc2));
        }
    }
    __syncthreads();
    GF_STAMP(4);

    // ---- K loop.  MATS = 2: warp = (matrix, n-tiles 2 ntp, 2 ntp + 1);  MATS = 1: warp = n-tile.
    constexpr int NPW = MATS == 2 ? 2 : 1;
    const int mat = MATS == 2 ? warp >> 2 : 0;
    const int nt0 = MATS == 2 ? (warp & 3) * 2 : warp;
    const bool two_sets = SETS == 2 && nmem > 8;
    float acc[NPW][SETS][4];
#pragma unroll
    for (int n = 0; n < NPW; ++n)
#pragma unroll
        for (int s = 0; s < SETS; ++s)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[n][s][c] = 0.f;

#pragma unroll 1
    for (int g = 0; g < NG; ++g) {
        // B operands of the group's 8 mma: the 16 activations k = 64 g + 16 T .. + 15 of member G (set 0) and member
        // 8 + G (set 1).  mma number 2t + h takes (x_k, 0), (x_k+1, 0) with k = 64 g + 16 T + 8 h + 2 t.
        uint32_t bp[SETS][8];                       // PACKED: word 4h + t holds (x_k, x_k+1)
        uint2 b1[8];                                // otherwise: entry 2t + h holds the two ready operands
        if (PACKED) {
#pragma unroll
            for (int s = 0; s < SETS; ++s) {
                const uint4 *ar = reinterpret_cast<const uint4 *>(asm_ + ((size_t)mat * SETS * 8 + s * 8 + G) * AST + g * 32 + 8 * T);
                const uint4 lo = ar[0], hi = ar[1];
                bp[s][0] = lo.x; bp[s][1] = lo.y; bp[s][2] = lo.z; bp[s][3] = lo.w;
                bp[s][4] = hi.x; bp[s][5] = hi.y; bp[s][6] = hi.z; bp[s][7] = hi.w;
            }
        } else {
            const uint32_t *ar = asm_ + ((size_t)mat * SETS * 8 + G) * AST + g * 64 + 2 * T;
#pragma unroll
            for (int m = 0; m < 8; ++m) b1[m] = *reinterpret_cast<const uint2 *>(ar + m * 8);
        }
        if (!mbar_wait(bars + g, 0, a.status)) { ok = false; break; }
        if (g == 0) GF_STAMP(5);
        const unsigned char *wrow = wsm + ((size_t)mat * KTC + 4 * g + T) * GEMV_WROW + nt0 * 128 + G * 16;
#pragma unroll
        for (int n = 0; n < ((GF_PROBE & 1) ? 0 : NPW); ++n) {
            const uint4 wv = *reinterpret_cast<const uint4 *>(wrow + n * 128);
            const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
            const uint32_t before = __shfl_sync(0xffffffffu, wv.w, (lane + 28) & 31);   // word 4G-1 (circular)
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const uint32_t pw = t == 0 ? before : w[t - 1];
                uint32_t uu[4];
                uu[0] = __funnelshift_r(w[t], pw, 12);
                uu[1] = __funnelshift_r(w[t], pw, 8);
                uu[2] = __funnelshift_r(w[t], pw, 4);
                uu[3] = w[t];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t x0, x1, x2, x3, af[4];
                    codeword_pair(uu[2 * h], x0, x1);        // k = 2t + 8h:     columns G, G + 8
                    codeword_pair(uu[2 * h + 1], x2, x3);    // k = 2t + 8h + 1: columns G, G + 8
                    af[0] = weight_dup(x0); af[1] = weight_dup(x1); af[2] = weight_dup(x2); af[3] = weight_dup(x3);
                    if (!PACKED) {
                        mma16816(acc[n][0], af, b1[2 * t + h].x, b1[2 * t + h].y);
                    } else {
                        const uint32_t bw0 = bp[0][4 * h + t];
                        mma16816(acc[n][0], af, bw0 & 0xffffu, bw0 >> 16);
                    }
                    if (SETS == 2 && two_sets) {
                        const uint32_t bw1 = bp[SETS - 1][4 * h + t];
                        mma16816(acc[n][SETS - 1], af, bw1 & 0xffffu, bw1 >> 16);
                    }
                }
            }
        }
    }
    if (!ok && lane == 0) atomicExch(a.status, GF_STATUS_TMA_TIMEOUT);
    if (GF_PROBE & 2) {
        if (acc[0][0][0] == 123.f) a.y[0] = acc[NPW - 1][0][1];
        return 0;
    }
    GF_STAMP(6);
    __syncthreads();                                // wsm is dead: part aliases it
    GF_STAMP(7);

    // ---- this split's partial[matrix][member][column] in shared memory, visible to the cluster
#pragma unroll
    for (int n = 0; n < NPW; ++n)
#pragma unroll
        for (int s = 0; s < SETS; ++s) {
            const int col = (nt0 + n) * 16 + G, mem = s * 8 + 2 * T;
            float *pp = part + ((size_t)mat * SETS * 8 + mem) * GEMV_PST + col;
            pp[0] = acc[n][s][0];
            pp[GEMV_PST] = acc[n][s][1];
            pp[8] = acc[n][s][2];
            pp[GEMV_PST + 8] = acc[n][s][3];
        }
    cluster_sync();
    GF_STAMP(8);

    // ---- member m is finished by CTA m % SK: the splits' partials are read from the peers' shared memory (all reads
    //      of a matrix in one batch, one round trip) and added in ascending split order, then the epilogue runs.
    auto reduce_splits = [&](int plane_row, float (&v)[4]) {
        float4 q[GEMV_MAX_SPLITS];
#pragma unroll
        for (int s = 0; s < GEMV_MAX_SPLITS; ++s)
            if (s < a.SK) q[s] = *reinterpret_cast<const float4 *>(cluster_map(part, s) + (size_t)plane_row * GEMV_PST + 4 * lane);
#pragma unroll
        for (int s = 0; s < GEMV_MAX_SPLITS; ++s)
            if (s < a.SK) { v[0] += q[s].x; v[1] += q[s].y; v[2] += q[s].z; v[3] += q[s].w; }
    };
    if (MATS == 2) {
        // Two warps per member, side by side: the odd warp sums and transforms the up matrix and hands the clamped
        // values over through shared memory, the even warp does the same for gate, applies SwiGLU, rotates for the down
        // projection and stores.  The single-member case (one token) is a serial tail of the whole kernel: this halves it.
        __shared__ __align__(16) float up_sh[GEMV_THREADS / 64][128];
        const int pw = warp >> 1, role = warp & 1;
        for (int m = split + a.SK * pw; m < nmem; m += a.SK * (GEMV_THREADS / 64)) {
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            reduce_splits(role * SETS * 8 + m, v);
            if (role == 0) GF_STAMP(11);
            fwht128(v, lane);
            if (role == 1) {
                float4 uu;
                uu.x = fminf(fmaxf(bf16r(v[0] * HAD_SCALE * scale_sh[1][4 * lane]), -a.limit), a.limit);
                uu.y = fminf(fmaxf(bf16r(v[1] * HAD_SCALE * scale_sh[1][4 * lane + 1]), -a.limit), a.limit);
                uu.z = fminf(fmaxf(bf16r(v[2] * HAD_SCALE * scale_sh[1][4 * lane + 2]), -a.limit), a.limit);
                uu.w = fminf(fmaxf(bf16r(v[3] * HAD_SCALE * scale_sh[1][4 * lane + 3]), -a.limit), a.limit);
                *reinterpret_cast<float4 *>(&up_sh[pw][4 * lane]) = uu;
                pair_barrier(pw);                                                // up values are there
            } else {
                float sg[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float gg = fminf(bf16r(v[j] * HAD_SCALE * scale_sh[0][4 * lane + j]), a.limit);
                    sg[j] = bf16r(gg / (1.f + expf(-gg)));
                }
                pair_barrier(pw);
                const float4 uu = *reinterpret_cast<const float4 *>(&up_sh[pw][4 * lane]);
                float o[4];
                o[0] = bf16r(sg[0] * uu.x) * scale_sh[2][4 * lane];
                o[1] = bf16r(sg[1] * uu.y) * scale_sh[2][4 * lane + 1];
                o[2] = bf16r(sg[2] * uu.z) * scale_sh[2][4 * lane + 2];
                o[3] = bf16r(sg[3] * uu.w) * scale_sh[2][4 * lane + 3];
                GF_STAMP(12);
                fwht128(o, lane);
                __half2 h01 = __halves2half2(__float2half_rn(o[0] * HAD_SCALE), __float2half_rn(o[1] * HAD_SCALE));
                __half2 h23 = __halves2half2(__float2half_rn(o[2] * HAD_SCALE), __float2half_rn(o[3] * HAD_SCALE));
                uint2 pk = make_uint2(*reinterpret_cast<uint32_t *>(&h01), *reinterpret_cast<uint32_t *>(&h23));
                *reinterpret_cast<uint2 *>(a.xd + (size_t)rows_sh[m] * a.N + nb * 128 + 4 * lane) = pk;
            }
            pair_barrier(pw);                                                    // up_sh may be written again
        }
    } else {
        for (int m = split + a.SK * warp; m < nmem; m += a.SK * (GEMV_THREADS / 32)) {
            const int p = rows_sh[m];
            const int n0 = nb * 128 + 4 * lane;
            float v0[4] = {0.f, 0.f, 0.f, 0.f};
            reduce_splits(m, v0);
            GF_STAMP(11);
            fwht128(v0, lane);
            float4 o;
            o.x = v0[0] * HAD_SCALE * scale_sh[0][4 * lane];
            o.y = v0[1] * HAD_SCALE * scale_sh[0][4 * lane + 1];
            o.z = v0[2] * HAD_SCALE * scale_sh[0][4 * lane + 2];
            o.w = v0[3] * HAD_SCALE * scale_sh[0][4 * lane + 3];
            if (a.mode == GEMV_LINEAR) {
                __half2 h01 = __halves2half2(__float2half_rn(o.x), __float2half_rn(o.y));
                __half2 h23 = __halves2half2(__float2half_rn(o.z), __float2half_rn(o.w));
                uint2 pk = make_uint2(*reinterpret_cast<uint32_t *>(&h01), *reinterpret_cast<uint32_t *>(&h23));
                *reinterpret_cast<uint2 *>(a.xd + (size_t)p * a.N + n0) = pk;
            } else {
                *reinterpret_cast<float4 *>(a.y + (size_t)p * a.N + n0) = o;
            }
        }
    }
    GF_STAMP(9);
    cluster_sync();                                 // peers may still be reading this CTA's partials
    GF_STAMP(10);
    return 0;
}

// One item per cluster: grid (N / 128, SK, distinct-expert bound), cluster (1, SK, 1).  (A persistent form, in which a
// resident set of clusters walks the item list, measured slower: clusters that start together stay in lock step, so
// the fetch, decode and exchange phases of the CTAs sharing an SM stop overlapping.)
template <int MATS, int SETS>
__global__ void __launch_bounds__(GEMV_THREADS, 4) gemv_kernel(const GemvArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    gemv_item<MATS, SETS>(a, smem, blockIdx.x, blockIdx.y, blockIdx.z);
}

// Input rotation (upstream rot_in_kernel, native/exl3.cu:224-241): one warp per (pair, 128-block, matrix);
// out[mat][p][blk] = fp16(H(x[row] * suh[mat][e]) / sqrt(128)).  IN = __nv_bfloat16 (layer input) or __half.
// picks == nullptr: pair p is row p of expert 0 (the single-linear probe).
template <typename IN>
__global__ void __launch_bounds__(256) rot_in_kernel(const IN *__restrict__ x, int x_stride, const int *__restrict__ picks,
                                                     const __half *__restrict__ suh0, const __half *__restrict__ suh1,
                                                     __half *__restrict__ out0, __half *__restrict__ out1, int K, int slots,
                                                     int P, int mats, int E, int shared_exl3, int e_lo, int e_hi) {
    // Wait first, trigger second: the kernel after this one reads the grouping tables in its prologue, before its own
    // wait, so it may only start once everything before this kernel (the grouping, the producer of x) has completed.
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KB = K >> 7;
    const long item = (long)blockIdx.x * 8 + warp;
    if (item >= (long)P * KB * mats) return;
    const int blk = (int)(item % KB);
    const int p = (int)((item / KB) % P), mat = (int)(item / ((long)KB * P));
    int row = p, e = 0;
    if (picks) {
        row = p / slots;
        e = picks[p];
        if (expert_skipped(e, E, shared_exl3, e_lo, e_hi)) return;
    }
    const __half *suh = (mat ? suh1 : suh0) + (size_t)e * K + blk * 128 + 4 * lane;
    const IN *xr = x + (size_t)row * x_stride + blk * 128 + 4 * lane;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = (float)xr[j] * __half2float(suh[j]);
    fwht128(v, lane);
    __half *o = (mat ? out1 : out0) + (size_t)p * K + blk * 128 + 4 * lane;
    __half2 h01 = __halves2half2(__float2half_rn(v[0] * HAD_SCALE), __float2half_rn(v[1] * HAD_SCALE));
    __half2 h23 = __halves2half2(__float2half_rn(v[2] * HAD_SCALE), __float2half_rn(v[3] * HAD_SCALE));
    *reinterpret_cast<uint2 *>(o) = make_uint2(*reinterpret_cast<uint32_t *>(&h01), *reinterpret_cast<uint32_t *>(&h23));
}

// Host-side launch helpers (defined in experts.cu).
int launch_rot_in(cudaStream_t s, const void *x, bool x_is_bf16, int x_stride, const int *picks, const __half *suh0,
                  const __half *suh1, __half *out0, __half *out1, int K, int slots, int P, int mats, int E,
                  int shared_exl3, int e_lo, int e_hi, bool pdl);
int launch_gemv(cudaStream_t s, int mats, GemvArgs a, int umax, bool pdl);

}  // namespace gf
