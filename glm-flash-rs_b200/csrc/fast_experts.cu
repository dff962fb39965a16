// FastExperts: the prefill owner (upstream src/fast_experts.rs:27-208) as two persistent grouped GEMMs on the
// 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory), sm_100a only.
//
// Replaces upstream's fast_rot_in / fast_expert_plan / fast_gu_shared / fast_gu_separate / fast_down /
// fast_down_large (native/exl3_prefill.cu:402-430,657-889), which decode each 16x16 trellis tile into mma.sync
// fragments in registers.  Here:
//
//   plan      one block: members per distinct expert, 128-row M tiles per expert, and the GROUPED row order
//             (rows of an expert contiguous): src_pair[j] = pair index of grouped row j.  Work items are
//             (expert, PAIR of M tiles, 128-column block); an expert with an odd tile count ends with a single.
//             Pairs come first in the item list, so that the static round-robin over CTAs is balanced.
//   rot       the input rotation writes Xs[j] = fp16(H(x[row] * suh[e]) / sqrt 128) in grouped order, so the A
//             operand of every M tile is a contiguous 128 x K slab that one TMA tensor load brings into shared
//             memory in the 128-byte-swizzled K-major layout the tensor core reads.
//   gemm      persistent CTAs, one per SM, 28 warps:
//               warp 0       TMA producer of the A stages (two M tiles of 128 rows x 64 k)
//               warp 1       issues tcgen05.mma (M 128 x N 128 x K 16, fp16 -> fp32), commits stages and passes
//               warp 2       allocates / frees tensor memory (512 columns)
//               warps 4-11   epilogue, one accumulator row per thread (tile 0: warps 4-7, tile 1: warps 8-11):
//                            tcgen05.ld 128 fp32, the 128-point Hadamard transform in the thread's registers,
//                            scales, limited SwiGLU, down-input rotation; fp16 Xd rows (gate/up) or fp32 Y rows (down)
//               warps 12-27  decode the trellis tiles of B (the weights) to fp16 straight into the swizzled K-major
//                            shared-memory tile (bit-exact codebook; conflict-free 32-bit stores); the packed words
//                            of the next stage are already in registers while a stage is decoded
//             A decoded B stage serves BOTH M tiles of the item (256 rows), which halves the decode work per
//             flop.  The gate and the up projection of an item are two PASSES over K with their own accumulators
//             (2 x 128 columns each): while the up pass runs, the epilogue warps turn the gate accumulators into
//             silu(gate) (kept as bf16 in shared memory), and the up pass's epilogue overlaps the next item's gate
//             pass, so tensor memory is double-buffered by construction.  Down is one pass per item, alternating
//             the two accumulator halves.  setmaxnreg moves registers from the producer and decode warpgroups to
//             the epilogue warpgroups.
// Arithmetic: one full-K fp32 accumulation chain per output (as upstream's prefill path, which is likewise not
// bit-equal to its decode path: native/exl3_prefill.cu:20-23), the same transforms and rounding points as
// upstream's epilogue (native/exl3_prefill.cu:596-622 == native/exl3.cu:260-321) with exp / divide in their fast
// forms.  Deterministic: static work assignment, no atomics; every pair's result depends only on its own row.
// Every wait is bounded; a wait that gives up raises the abort flag, every role leaves its loops, tensor memory
// is freed and the status word reports the failure.
#include <cuda.h>

#include <algorithm>
#include <new>

#include "gemv.cuh"

namespace gf {
int check_config(const glmflash_config *cfg, size_t cfg_bytes, int max_rows_limit);

// FG_PROBE (timing experiments only, wrong results): 1 = decode warps store the raw words instead of decoding,
// 2 = epilogue warps skip their arithmetic, 4 = no packed-word loads (decode a constant).
#ifndef FG_PROBE
#define FG_PROBE 0
#endif
// FG_DEC_WARPS: trellis-decode warps per CTA (8 or 16).  With 16 (the default: the decode is what the kernel waits for,
// and four instead of two decode warps per scheduler raise its issue rate; measured 0.90 -> 0.80 ms per layer) every
// warp owns two n-tiles of a k-tile instead of four, the CTA has 896 threads, and the register pool (896 x 72) is
// split 24 / 152 / 40 per thread over the producer, epilogue and decode warpgroups (8 warps: 40 / 152 / 64 of 640 x 96).
#ifndef FG_DEC_WARPS
#define FG_DEC_WARPS 16
#endif
#ifndef FG_EPI_REGS
#define FG_EPI_REGS 152
#endif
#ifndef FG_DEC_REGS
#define FG_DEC_REGS 40
#endif
#define FG_STR2(x) #x
#define FG_STR(x) FG_STR2(x)
constexpr int FG_THREADS = (12 + FG_DEC_WARPS) * 32;
constexpr int FG_BM = 128, FG_BN = 128, FG_BK = 64;
constexpr int FG_TILE_BYTES = FG_BM * FG_BK * 2;           // 16 KB: one 128 x 64 fp16 operand tile
constexpr int FG_MAXU = 1024;

// plan layout (int32): [0] total M tiles, [1] total grouped rows, [2] pair items, [3] single items,
// then three prefix arrays of FG_MAXU + 1 entries: pair_base, single_base, row_base
constexpr int PLAN_PAIR_BASE = 4, PLAN_SINGLE_BASE = PLAN_PAIR_BASE + FG_MAXU + 1,
              PLAN_ROW_BASE = PLAN_SINGLE_BASE + FG_MAXU + 1, PLAN_INTS = PLAN_ROW_BASE + FG_MAXU + 1;

// ---------------------------------------------------------------------------------------------- plan
// Launched with one block per bank entry: every block recomputes the (tiny) scans, block 0 publishes the plan,
// block b writes the grouped rows of distinct expert b.
__global__ void __launch_bounds__(FG_MAXU) fast_plan_kernel(const int *__restrict__ ids, const int *__restrict__ count,
                                                          const int *__restrict__ members, int maxm, int slots, int E,
                                                          int shared_exl3, int e_lo, int e_hi, int srow_lo, int srow_hi,
                                                          int *__restrict__ plan, int *__restrict__ src_pair,
                                                          int *__restrict__ row_expert) {
    __shared__ int cnt_sh[FG_MAXU], row_sh[FG_MAXU], e_sh[FG_MAXU], first_sh[FG_MAXU];
    __shared__ int wsum[4][32];
    const int u = threadIdx.x, lane = u & 31, warp = u >> 5;
    const int n = min(count[0], FG_MAXU);
    int cnt = 0, e = -1, first = 0;
    if (u < n) {
        e = ids[u];
        if (!expert_skipped(e, E, shared_exl3, e_lo, e_hi)) {
            const int *m = members + (size_t)u * maxm;
            int lo = 0, hi = maxm;                          // members come first: the count is the first -1
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (m[mid] >= 0) lo = mid + 1; else hi = mid;
            }
            cnt = lo;
            if (e == E && srow_hi > srow_lo) {
                // the shared expert is computed here for a window of rows only: members ascend by row (code = row * 32
                // + slot), so the window is a contiguous run of the list
                auto lower = [&](int row) {                 // first member whose row is >= `row`
                    int a = 0, b = cnt;
                    while (a < b) {
                        const int mid = (a + b) >> 1;
                        if ((m[mid] >> 5) < row) a = mid + 1; else b = mid;
                    }
                    return a;
                };
                first = lower(srow_lo);
                cnt = lower(srow_hi) - first;
            }
        }
    }
    const int tiles = (cnt + FG_BM - 1) / FG_BM;
    const int pairs = tiles >> 1, single = tiles & 1;
    // block-wide exclusive scans of pairs, singles, rows (and the tile total)
    int p_inc = pairs, s_inc = single, r_inc = cnt, t_inc = tiles;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int a = __shfl_up_sync(0xffffffffu, p_inc, d), b = __shfl_up_sync(0xffffffffu, s_inc, d),
                  c = __shfl_up_sync(0xffffffffu, r_inc, d), t = __shfl_up_sync(0xffffffffu, t_inc, d);
        if (lane >= d) { p_inc += a; s_inc += b; r_inc += c; t_inc += t; }
    }
    if (lane == 31) { wsum[0][warp] = p_inc; wsum[1][warp] = s_inc; wsum[2][warp] = r_inc; wsum[3][warp] = t_inc; }
    __syncthreads();
    int p_off = 0, s_off = 0, r_off = 0, p_all = 0, s_all = 0, r_all = 0, t_all = 0;
    for (int w = 0; w < 32; ++w) {
        if (w < warp) { p_off += wsum[0][w]; s_off += wsum[1][w]; r_off += wsum[2][w]; }
        p_all += wsum[0][w]; s_all += wsum[1][w]; r_all += wsum[2][w]; t_all += wsum[3][w];
    }
    const int p_ex = p_off + p_inc - pairs, s_ex = s_off + s_inc - single, r_ex = r_off + r_inc - cnt;
    cnt_sh[u] = cnt; row_sh[u] = r_ex; e_sh[u] = e; first_sh[u] = first;
    if (blockIdx.x == 0) {
        plan[PLAN_PAIR_BASE + u] = p_ex;
        plan[PLAN_SINGLE_BASE + u] = s_ex;
        plan[PLAN_ROW_BASE + u] = r_ex;
    }
    if (u == 0 && blockIdx.x == 0) {
        plan[0] = t_all; plan[1] = r_all; plan[2] = p_all; plan[3] = s_all;
        plan[PLAN_PAIR_BASE + FG_MAXU] = p_all;
        plan[PLAN_SINGLE_BASE + FG_MAXU] = s_all;
        plan[PLAN_ROW_BASE + FG_MAXU] = r_all;
    }
    __syncthreads();
    for (int uu = blockIdx.x; uu < n; uu += gridDim.x) {
        const int c = cnt_sh[uu], rb = row_sh[uu], ee = e_sh[uu], f0 = first_sh[uu];
        for (int m = u; m < c; m += FG_MAXU) {
            const int code = members[(size_t)uu * maxm + f0 + m];
            src_pair[rb + m] = (code >> 5) * slots + (code & 31);
            row_expert[rb + m] = ee;
        }
    }
}

// ---------------------------------------------------------------------------------------------- rotation
// One CTA (8 warps) per grouped row: the row's expert and source row are looked up once, every warp rotates
// K/128/8 blocks, for one (shared_x) or both input scale vectors.
__global__ void __launch_bounds__(256) fast_rot_kernel(const __nv_bfloat16 *__restrict__ x, int x_stride,
                                                       const int *__restrict__ plan, const int *__restrict__ src_pair,
                                                       const int *__restrict__ row_expert, const __half *__restrict__ suh0,
                                                       const __half *__restrict__ suh1, __half *__restrict__ out0,
                                                       __half *__restrict__ out1, int K, int slots, int mats) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KB = K >> 7, rows = plan[1];
    for (int j = blockIdx.x; j < rows; j += gridDim.x) {
        const int p = src_pair[j], e = row_expert[j], row = p / slots;
        // two 128-blocks of the warp per round: all their loads are issued before the first transform
        for (int blk0 = warp; blk0 < KB; blk0 += 16) {
            const int n2 = blk0 + 8 < KB ? 2 : 1;
            uint2 xv[2], sv[2][2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (i >= n2) break;
                const int k = (blk0 + 8 * i) * 128 + 4 * lane;
                xv[i] = *reinterpret_cast<const uint2 *>(x + (size_t)row * x_stride + k);
#pragma unroll
                for (int mat = 0; mat < 2; ++mat)
                    if (mat < mats) sv[i][mat] = __ldg(reinterpret_cast<const uint2 *>((mat ? suh1 : suh0) + (size_t)e * K + k));
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (i >= n2) break;
                const int k = (blk0 + 8 * i) * 128 + 4 * lane;
                const __nv_bfloat162 x01 = *reinterpret_cast<const __nv_bfloat162 *>(&xv[i].x),
                                     x23 = *reinterpret_cast<const __nv_bfloat162 *>(&xv[i].y);
                const float xf[4] = {__bfloat162float(x01.x), __bfloat162float(x01.y), __bfloat162float(x23.x), __bfloat162float(x23.y)};
#pragma unroll
                for (int mat = 0; mat < 2; ++mat) {
                    if (mat >= mats) break;
                    const __half2 s01 = *reinterpret_cast<const __half2 *>(&sv[i][mat].x),
                                  s23 = *reinterpret_cast<const __half2 *>(&sv[i][mat].y);
                    float v[4] = {xf[0] * __low2float(s01), xf[1] * __high2float(s01), xf[2] * __low2float(s23), xf[3] * __high2float(s23)};
                    fwht128(v, lane);
                    __half2 h01 = __halves2half2(__float2half_rn(v[0] * HAD_SCALE), __float2half_rn(v[1] * HAD_SCALE));
                    __half2 h23 = __halves2half2(__float2half_rn(v[2] * HAD_SCALE), __float2half_rn(v[3] * HAD_SCALE));
                    *reinterpret_cast<uint2 *>((mat ? out1 : out0) + (size_t)j * K + k) =
                        make_uint2(*reinterpret_cast<uint32_t *>(&h01), *reinterpret_cast<uint32_t *>(&h23));
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------- tcgen05 helpers
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t *slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_smem)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]^T, M 128 x N 128 x K 16, fp16 operands, fp32 accumulate
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive on an mbarrier when every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float *v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart; the tile base is 1024-aligned and
// a K step of 16 halves advances the start address by 32 bytes inside the swizzle atom.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);          // start address
    d |= (uint64_t)1 << 16;                               // leading byte offset (unused with swizzle): 16 B
    d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset: 8 rows x 128 B
    d |= (uint64_t)1 << 46;                               // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                               // SWIZZLE_128B
    return d;
}
// kind::f16: D fp32, A and B fp16, both K-major, N 128, M 128
constexpr uint32_t UMMA_IDESC = (1u << 4) | ((uint32_t)(FG_BN >> 3) << 17) | ((uint32_t)(FG_BM >> 4) << 24);

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// Wait on an mbarrier phase, giving up when the abort flag is up or after a bounded number of polls.
__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    for (uint32_t i = 0; i < 400000u; ++i) {                  // each poll may sleep up to 10 us: at most about 4 s
        if (mbar_try_wait_hint(bar, parity, 10000u)) return true;
        if (*abort_flag) return false;
        // another CTA of this launch has already given up: leave as well instead of sitting out the limit here too
        if ((i & 15u) == 15u && *reinterpret_cast<volatile int *>(status) != 0) { *abort_flag = 1; return false; }
    }
    *abort_flag = 1;
    atomicExch(status, code);
    return false;
}

// In-register 128-point Walsh-Hadamard transform, butterflies stride 1..64, (lower + upper, lower - upper):
// upstream's order (native/exl3.cu:208-219), so every sum associates as there.
// Two values rounded to bf16 (nearest even) by one packed conversion, read back as fp32: per value the bits of bf16r.
__device__ __forceinline__ float2 bf16r2(float x, float y) {
    const __nv_bfloat162 b = __float22bfloat162_rn(make_float2(x, y));
    const uint32_t w = *reinterpret_cast<const uint32_t *>(&b);
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
// From stride 2 on, the two neighbours (i, i + 1) take the same side of their butterflies, so a pair goes through one
// packed fp32 instruction of sm_100 (add.f32x2 / fma.f32x2; a - b as b * -1 + a, one rounding, the same bits): half
// the issue slots of the transform, which matters because this kernel is bound by instruction issue.
__device__ __forceinline__ void fwht128_regs(float (&v)[128]) {
#pragma unroll
    for (int i = 0; i < 128; i += 2) {
        const float a = v[i], b = v[i + 1];
        v[i] = a + b;
        v[i + 1] = a - b;
    }
    const float2 neg1 = make_float2(-1.f, -1.f);
#pragma unroll
    for (int s = 2; s < 128; s <<= 1)
#pragma unroll
        for (int i = 0; i < 128; i += 2)
            if (!(i & s)) {
                const float2 a = make_float2(v[i], v[i + 1]), b = make_float2(v[i | s], v[(i | s) + 1]);
                const float2 lo = __fadd2_rn(a, b), hi = __ffma2_rn(b, neg1, a);
                v[i] = lo.x; v[i + 1] = lo.y;
                v[i | s] = hi.x; v[(i | s) + 1] = hi.y;
            }
}

struct FastGemmArgs {
    const uint32_t *T0, *T1;       // trellis banks of pass 0 / pass 1 (gate, up;  down: T0 only)
    const int *ids, *plan, *src_pair;
    const __half *sv0, *sv1, *sd;  // gate/up: svh_g, svh_u, suh_d;  down: svh_d
    __half *xd;                    // gate/up out, grouped rows [rows][N]
    float *y;                      // down out, pair rows [P][N]
    int *status;
    int K, N, shared_x;
    float limit;
};

// One work item: expert u (id e), its M tiles tile0 (and tile0 + 1 when ntiles == 2) starting at grouped row row0,
// cnt0 / cnt1 valid rows in them, column block nb.
struct ItemInfo {
    int e, row0, cnt0, cnt1, ntiles, nb;
};
__device__ __forceinline__ int last_le(const int *base, int n, int v) {     // largest i < n with base[i] <= v
    int lo = 0, hi = n;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (base[mid] <= v) lo = mid; else hi = mid;
    }
    return lo;
}
__device__ __forceinline__ ItemInfo item_info(int item, int NB, int pairs_all, const int *pair_base, const int *single_base,
                                              const int *row_base, const int *ids) {
    ItemInfo t;
    const int q = item / NB;
    t.nb = item % NB;
    int u, tile0;
    if (q < pairs_all) {
        u = last_le(pair_base, FG_MAXU, q);
        tile0 = 2 * (q - pair_base[u]);
        t.ntiles = 2;
    } else {
        u = last_le(single_base, FG_MAXU, q - pairs_all);
        const int cnt = row_base[u + 1] - row_base[u];
        tile0 = (cnt + FG_BM - 1) / FG_BM - 1;
        t.ntiles = 1;
    }
    const int cnt = row_base[u + 1] - row_base[u];
    t.e = ids[u];
    t.row0 = row_base[u] + tile0 * FG_BM;
    t.cnt0 = min(FG_BM, cnt - tile0 * FG_BM);
    t.cnt1 = t.ntiles == 2 ? min(FG_BM, cnt - (tile0 + 1) * FG_BM) : 0;
    return t;
}

template <int MATS>
struct FgCfg {
    static constexpr int STAGES = MATS == 2 ? 3 : 4;
    static constexpr int STAGE_BYTES = 3 * FG_TILE_BYTES;                                    // A tile 0, A tile 1, B
    static constexpr int GBUF_BYTES = MATS == 2 ? 64 * 256 * 4 : 0;                          // silu(gate) as bf16 pairs
    static constexpr int TABLE_BYTES = (256 + 3 * 128 * 4 + 2 * (FG_MAXU + 1) * 4 + 64 + 127) / 128 * 128;   // keeps tbuf 128-byte aligned
    static constexpr int TBUF_BYTES = MATS == 1 ? 8 * 32 * 16 * 4 : 0;        // down: per epilogue warp 32 rows x 16 floats
    static constexpr size_t SMEM = 1024 /*align*/ + (size_t)STAGES * STAGE_BYTES + GBUF_BYTES + TABLE_BYTES + TBUF_BYTES;
};

template <int MATS>
__global__ void __launch_bounds__(FG_THREADS, 1)
fast_gemm_kernel(const __grid_constant__ CUtensorMap mapA0, const __grid_constant__ CUtensorMap mapA1, const FastGemmArgs a) {
    using C = FgCfg<MATS>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);      // 1024-aligned operand tiles
    unsigned char *stages = smem;
    uint32_t *gbuf = reinterpret_cast<uint32_t *>(smem + (size_t)C::STAGES * C::STAGE_BYTES); // [64][256]
    unsigned char *tables = smem + (size_t)C::STAGES * C::STAGE_BYTES + C::GBUF_BYTES;
    uint64_t *full = reinterpret_cast<uint64_t *>(tables);                 // [STAGES] A landed (tx) + the decode warps
    uint64_t *empty = full + C::STAGES;                                    // [STAGES] MMAs of the stage completed
    uint64_t *tmem_full = empty + C::STAGES;                               // [2] accumulators of a pass complete
    uint64_t *tmem_empty = tmem_full + 2;                                  // [2] accumulators drained (8 epilogue warps)
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float *scales = reinterpret_cast<float *>(tables + 256);               // [3][128]
    int *pair_base = reinterpret_cast<int *>(tables + 256 + 3 * 128 * 4);  // [FG_MAXU + 1]
    int *single_base = pair_base + FG_MAXU + 1;                            // [FG_MAXU + 1]
    float *tbuf = reinterpret_cast<float *>(tables + C::TABLE_BYTES);      // [8 warps][32 rows][16] (down only)
    const int *row_base = a.plan + PLAN_ROW_BASE;                          // global (L1 / L2 hits)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int KT = a.K >> 4, NTILES = a.N >> 4, NB = a.N >> 7, KS = a.K / FG_BK;
    const int pairs_all = a.plan[2];
    const int total = (pairs_all + a.plan[3]) * NB;

    if (tid == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(full + s, 1 + FG_DEC_WARPS); mbar_init(empty + s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tmem_full + b, 1); mbar_init(tmem_empty + b, 8); }
        *abort_flag = 0;
        mbar_fence_init();
    }
    for (int i = tid; i <= FG_MAXU; i += FG_THREADS) {
        pair_base[i] = a.plan[PLAN_PAIR_BASE + i];
        single_base[i] = a.plan[PLAN_SINGLE_BASE + i];
    }
    if (warp == 2) tmem_alloc(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 4) {
        // ------------------------------------------------------------------ warpgroup 0: TMA, MMA issue
#if FG_DEC_WARPS == 16
        asm volatile("setmaxnreg.dec.sync.aligned.u32 24;");
#else
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
#endif
        if (warp == 0 && lane == 0) {
            uint32_t it = 0;
            for (int item = blockIdx.x; item < total && !*abort_flag; item += gridDim.x) {
                const ItemInfo t = item_info(item, NB, pairs_all, pair_base, single_base, row_base, a.ids);
                bool ok = true;
                for (int pm = 0; pm < MATS && ok; ++pm) {
                    const CUtensorMap *map = (pm == 1 && !a.shared_x) ? &mapA1 : &mapA0;
                    for (int s = 0; s < KS; ++s, ++it) {
                        const int slot = it % C::STAGES;
                        const uint32_t n = it / C::STAGES;
                        if (!wait_or_abort(empty + slot, (n & 1) ^ 1, abort_flag, a.status, GF_STATUS_TMA_TIMEOUT)) { ok = false; break; }
                        unsigned char *st = stages + (size_t)slot * C::STAGE_BYTES;
                        if (FG_PROBE & 16) { mbar_arrive(full + slot); continue; }   // no A loads
                        mbar_expect_tx(full + slot, t.ntiles * FG_TILE_BYTES);
                        tma_load_2d(st, map, s * FG_BK, t.row0, full + slot);
                        if (t.ntiles == 2) tma_load_2d(st + FG_TILE_BYTES, map, s * FG_BK, t.row0 + FG_BM, full + slot);
                    }
                }
                if (!ok) break;
            }
        } else if (warp == 1 && lane == 0) {
            // One thread issues every MMA.  Its own instruction stream is the critical path of the tensor pipe, so the
            // shared-memory descriptors are built once (stage 0) and advanced by adding constants: the address field
            // counts 16-byte units, a stage is STAGE_BYTES apart, a K step of 16 halves is 32 bytes.
            const uint64_t desc_a0 = umma_desc_sw128(smem_u32(stages));
            const uint64_t desc_b0 = umma_desc_sw128(smem_u32(stages) + 2 * FG_TILE_BYTES);
            uint32_t it = 0, pc = 0;
            for (int item = blockIdx.x; item < total && !*abort_flag; item += gridDim.x) {
                const ItemInfo t = item_info(item, NB, pairs_all, pair_base, single_base, row_base, a.ids);
                const bool two = t.ntiles == 2;
                bool ok = true;
                for (int pm = 0; pm < MATS && ok; ++pm, ++pc) {
                    const uint32_t pb = pc & 1;
                    if (!wait_or_abort(tmem_empty + pb, ((pc >> 1) & 1) ^ 1, abort_flag, a.status, GF_STATUS_MMA_TIMEOUT)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t d0 = tmem_base + pb * 256;
                    for (int s = 0; s < KS; ++s, ++it) {
                        const uint32_t slot = it % C::STAGES;
                        const uint32_t n = it / C::STAGES;
                        if (!wait_or_abort(full + slot, n & 1, abort_flag, a.status, GF_STATUS_MMA_TIMEOUT)) { ok = false; break; }
                        tc_fence_after();
                        const uint64_t da = desc_a0 + (uint64_t)(slot * (C::STAGE_BYTES >> 4));
                        const uint64_t db = desc_b0 + (uint64_t)(slot * (C::STAGE_BYTES >> 4));
                        const uint32_t acc0 = s > 0 ? 1u : 0u;
                        if (two) {
#pragma unroll
                            for (int kk = 0; kk < FG_BK / 16; ++kk) {
                                umma_f16(d0, da + 2 * kk, db + 2 * kk, UMMA_IDESC, kk > 0 ? 1u : acc0);
                                umma_f16(d0 + FG_BN, da + (FG_TILE_BYTES >> 4) + 2 * kk, db + 2 * kk, UMMA_IDESC, kk > 0 ? 1u : acc0);
                            }
                        } else {
#pragma unroll
                            for (int kk = 0; kk < FG_BK / 16; ++kk)
                                umma_f16(d0, da + 2 * kk, db + 2 * kk, UMMA_IDESC, kk > 0 ? 1u : acc0);
                        }
                        umma_commit(empty + slot);          // the stage may be overwritten once these MMAs have read it
                    }
                    if (ok) umma_commit(tmem_full + pb);    // the accumulators of this pass are complete
                }
                if (!ok) break;
            }
        }
    } else if (warp < 12) {
        // ------------------------------------------------------------------ warpgroups 1-2: epilogue (tile 0 | tile 1)
#if FG_DEC_WARPS == 16
        asm volatile("setmaxnreg.inc.sync.aligned.u32 " FG_STR(FG_EPI_REGS) ";");
#else
        asm volatile("setmaxnreg.inc.sync.aligned.u32 152;");
#endif
        const int q = warp & 3, tl = (warp - 4) >> 2;        // TMEM lane quadrant, M tile of the item
        const int m = q * 32 + lane, em = tl * 128 + m;      // row of the tile, row of the item (0..255)
        uint32_t pc = 0;
        bool ok = true;
        // A warp whose wait gave up (or that sees the abort flag) does not leave this loop: it walks the remaining items
        // arriving at the two barriers only, so that a sibling which passed the same wait at the last moment never
        // stands alone at a barrier of eight warps.
        for (int item = blockIdx.x; item < total; item += gridDim.x) {
            const ItemInfo t = item_info(item, NB, pairs_all, pair_base, single_base, row_base, a.ids);
            const bool has = tl < t.ntiles;
            const int cnt = tl == 0 ? t.cnt0 : t.cnt1;
            // scale vectors of (expert, column block): written by the first 128 epilogue threads, read by all 256
            asm volatile("bar.sync 1, 256;");
            if (ok && *abort_flag) ok = false;
            if (ok && em < 128) {
                const size_t o = (size_t)t.e * a.N + t.nb * 128 + em;
                // the 1 / sqrt(128) of every Hadamard transform is folded into the scale vectors here (the transform is
                // linear), which takes one multiply per element out of each epilogue step
                scales[em] = __half2float(a.sv0[o]) * HAD_SCALE;
                if (MATS == 2) { scales[128 + em] = __half2float(a.sv1[o]) * HAD_SCALE; scales[256 + em] = __half2float(a.sd[o]) * HAD_SCALE; }
            }
            asm volatile("bar.sync 1, 256;");
            if (!ok) continue;
            float v[128];
            for (int pm = 0; pm < MATS; ++pm, ++pc) {
                const uint32_t pb = pc & 1;
                if (!wait_or_abort(tmem_full + pb, (pc >> 1) & 1, abort_flag, a.status, GF_STATUS_MMA_TIMEOUT)) { ok = false; break; }
                tc_fence_after();
                if (has) {
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + pb * 256 + tl * FG_BN;
#pragma unroll
                    for (int c = 0; c < 4; ++c) tmem_ld32(taddr + c * 32, v + c * 32);
                    tmem_ld_wait();
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tmem_empty + pb);             // this warp's rows are in registers
                if (!has) continue;
                if (FG_PROBE & 2) {
                    if (v[5] == 1.2345f && m < cnt) a.status[1] = 1;
                    continue;
                }
                fwht128_regs(v);
                const float2 *sc2 = reinterpret_cast<const float2 *>(scales);       // (8-byte aligned: the tables are 128-byte aligned)
                if (MATS == 2 && pm == 0) {
                    // gate: scale, bf16 rounding, clamp, silu (rounded) -> two bf16 per word, this thread's column of gbuf
#pragma unroll
                    for (int i = 0; i < 64; ++i) {
                        const float2 sg = sc2[i];
                        const float2 gr = bf16r2(v[2 * i] * sg.x, v[2 * i + 1] * sg.y);
                        const float g0 = fminf(gr.x, a.limit), g1 = fminf(gr.y, a.limit);
                        // (one packed conversion rounds both values to bf16 and packs them: .x in the low half)
                        const __nv_bfloat162 sp = __float22bfloat162_rn(make_float2(__fdividef(g0, 1.f + __expf(-g0)),
                                                                                   __fdividef(g1, 1.f + __expf(-g1))));
                        gbuf[i * 256 + em] = *reinterpret_cast<const uint32_t *>(&sp);
                    }
                } else if (MATS == 2) {
#pragma unroll
                    for (int i = 0; i < 64; ++i) {
                        const uint32_t gp = gbuf[i * 256 + em];
                        const float2 su = sc2[64 + i], sd2 = sc2[128 + i];
                        const float2 ur = bf16r2(v[2 * i] * su.x, v[2 * i + 1] * su.y);
                        const float u0 = fminf(fmaxf(ur.x, -a.limit), a.limit), u1 = fminf(fmaxf(ur.y, -a.limit), a.limit);
                        const float2 pr = bf16r2(__uint_as_float(gp << 16) * u0, __uint_as_float(gp & 0xffff0000u) * u1);
                        v[2 * i] = pr.x * sd2.x;
                        v[2 * i + 1] = pr.y * sd2.y;
                    }
                    fwht128_regs(v);
                    if (m < cnt) {
                        uint4 *o = reinterpret_cast<uint4 *>(a.xd + (size_t)(t.row0 + em) * a.N + t.nb * 128);
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            __half2 h[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j)       // one packed conversion per pair (the same rounding per value)
                                h[j] = __float22half2_rn(make_float2(v[8 * c + 2 * j], v[8 * c + 2 * j + 1]));
                            o[c] = make_uint4(*reinterpret_cast<uint32_t *>(&h[0]), *reinterpret_cast<uint32_t *>(&h[1]),
                                              *reinterpret_cast<uint32_t *>(&h[2]), *reinterpret_cast<uint32_t *>(&h[3]));
                        }
                    }
                } else {
                    // down: y rows are pair rows, scattered by src_pair.  A thread owns one row, so direct stores would
                    // put 32 rows x 16 bytes into every store instruction (half-filled sectors).  The rows go through a
                    // per-warp shared-memory tile, 16 columns at a time, and leave as 8 rows x 64 contiguous bytes per
                    // instruction.  Chunk c of row r sits at chunk c ^ ((r >> 1) & 3): conflict-free both ways.
                    const int p = m < cnt ? a.src_pair[t.row0 + em] : -1;
                    float *wbuf = tbuf + (warp - 4) * 512;
#pragma unroll
                    for (int ch = 0; ch < 8; ++ch) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const int col = ch * 16 + 4 * c;
                            const float4 s4 = *reinterpret_cast<const float4 *>(scales + col);
                            *reinterpret_cast<float4 *>(wbuf + lane * 16 + ((c ^ ((lane >> 1) & 3)) << 2)) =
                                make_float4(v[col] * s4.x, v[col + 1] * s4.y, v[col + 2] * s4.z, v[col + 3] * s4.w);
                        }
                        __syncwarp();
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int rr = (lane >> 2) + 8 * i, c = lane & 3;
                            const float4 val = *reinterpret_cast<const float4 *>(wbuf + rr * 16 + ((c ^ ((rr >> 1) & 3)) << 2));
                            const int pr = __shfl_sync(0xffffffffu, p, rr);              // pair row of warp row rr
                            if (pr >= 0)
                                *reinterpret_cast<float4 *>(a.y + (size_t)pr * a.N + t.nb * 128 + ch * 16 + 4 * c) = val;
                        }
                        __syncwarp();
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ warpgroups 3-4: trellis decode of B
#if FG_DEC_WARPS == 16
        asm volatile("setmaxnreg.dec.sync.aligned.u32 " FG_STR(FG_DEC_REGS) ";");
#else
        asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
#endif
        const int dw = warp - 12;
        constexpr int NTL = 32 / FG_DEC_WARPS;               // n tiles of this warp per stage (4 k-tiles x 8 n-tiles in all)
        const int ktl = dw & 3, nt_begin = (dw >> 2) * NTL;
        const int g = lane >> 2, tq = lane & 3;
        // byte offsets inside the B tile of this lane's four 32-bit stores (before the n-tile offset)
        const int c0 = 2 * ktl, c1 = 2 * ktl + 1;
        const int off_lo0 = nt_begin * 2048 + g * 128 + ((c0 ^ g) << 4) + 4 * tq;     // n = g,     k = 2t
        const int off_lo1 = nt_begin * 2048 + g * 128 + ((c1 ^ g) << 4) + 4 * tq;     // n = g,     k = 2t + 8
        uint32_t it = 0;
        bool ok = true;
        int item = blockIdx.x, pm = 0;
        ItemInfo t{};
        auto src_of = [&](const ItemInfo &ti, int pmat, int s) {
            return (pmat ? a.T1 : a.T0) + (((size_t)ti.e * KT + 4 * s + ktl) * NTILES + (size_t)ti.nb * 8 + nt_begin) * 32 + lane;
        };
        auto load_words = [&](const uint32_t *src, uint32_t (&w)[NTL]) {
#pragma unroll
            for (int i = 0; i < NTL; ++i) w[i] = (FG_PROBE & 4) ? (uint32_t)(size_t)src : __ldg(src + i * 32);
        };
        auto do_stage = [&](const uint32_t (&wr)[NTL]) {
            const int slot = it % C::STAGES;
            const uint32_t n = it / C::STAGES;
            if (!wait_or_abort(empty + slot, (n & 1) ^ 1, abort_flag, a.status, GF_STATUS_TMA_TIMEOUT)) { ok = false; return; }
            unsigned char *bt = stages + (size_t)slot * C::STAGE_BYTES + 2 * FG_TILE_BYTES;
#pragma unroll
            for (int i = 0; i < NTL; ++i) {
                const uint32_t w = wr[i];
                if (FG_PROBE & 8) continue;                    // no stores at all
                if (FG_PROBE & 1) {
                    unsigned char *tbp = bt + i * 2048;
                    *reinterpret_cast<uint32_t *>(tbp + off_lo0) = w;
                    *reinterpret_cast<uint32_t *>(tbp + off_lo1) = w;
                    *reinterpret_cast<uint32_t *>(tbp + off_lo0 + 1024) = w;
                    *reinterpret_cast<uint32_t *>(tbp + off_lo1 + 1024) = w;
                    continue;
                }
                const uint32_t pw = __shfl_sync(0xffffffffu, w, (lane + 31) & 31);
                uint32_t x0, x1, x2, x3, x4, x5, x6, x7;
                codeword_pair(__funnelshift_r(w, pw, 12), x0, x4);     // j = 0 | 4
                codeword_pair(__funnelshift_r(w, pw, 8), x1, x5);      // j = 1 | 5
                codeword_pair(__funnelshift_r(w, pw, 4), x2, x6);      // j = 2 | 6
                codeword_pair(w, x3, x7);                              // j = 3 | 7
                const uint32_t p01 = __byte_perm(weight_dup(x0), weight_dup(x1), 0x5410);
                const uint32_t p23 = __byte_perm(weight_dup(x2), weight_dup(x3), 0x5410);
                const uint32_t p45 = __byte_perm(weight_dup(x4), weight_dup(x5), 0x5410);
                const uint32_t p67 = __byte_perm(weight_dup(x6), weight_dup(x7), 0x5410);
                unsigned char *tb = bt + i * 2048;
                *reinterpret_cast<uint32_t *>(tb + off_lo0) = p01;
                *reinterpret_cast<uint32_t *>(tb + off_lo1) = p23;
                *reinterpret_cast<uint32_t *>(tb + off_lo0 + 1024) = p45;           // n = g + 8
                *reinterpret_cast<uint32_t *>(tb + off_lo1 + 1024) = p67;
            }
            fence_async_smem();                              // generic-proxy stores -> visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(full + slot);
            ++it;
        };
        // Packed words are fetched three stages ahead into four register buffers; KS is a multiple of 4, so the
        // buffer of a stage is s & 3 at compile time.  (pass, stage) + d stages ahead, across pass / item boundaries:
        uint32_t w0[NTL], w1[NTL], w2[NTL], w3[NTL];
        bool valid = item < total;
        int n_item = item, n_pm = 0;
        ItemInfo tn{};
        bool n_valid = false;
        auto fetch = [&](int s, uint32_t (&w)[NTL]) {          // stage s of the current pass; s >= KS: the next pass
            if (s < KS) load_words(src_of(t, pm, s), w);
            else if (n_valid) load_words(src_of(tn, n_pm, s - KS), w);
        };
        auto advance = [&]() {                                 // describe the pass after (item, pm)
            n_item = item; n_pm = pm + 1; tn = t; n_valid = true;
            if (n_pm == MATS) {
                n_pm = 0;
                n_item = item + gridDim.x;
                n_valid = n_item < total;
                if (n_valid) tn = item_info(n_item, NB, pairs_all, pair_base, single_base, row_base, a.ids);
            }
        };
        if (valid) {
            t = item_info(item, NB, pairs_all, pair_base, single_base, row_base, a.ids);
            advance();
            fetch(0, w0); fetch(1, w1); fetch(2, w2);
        }
        while (valid && ok && !*abort_flag) {
            for (int s = 0; s < KS && ok; s += 4) {
                fetch(s + 3, w3); do_stage(w0); if (!ok) break;
                fetch(s + 4, w0); do_stage(w1); if (!ok) break;
                fetch(s + 5, w1); do_stage(w2); if (!ok) break;
                fetch(s + 6, w2); do_stage(w3);
            }
            item = n_item; pm = n_pm; t = tn; valid = n_valid;
            if (valid) advance();
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 2) tmem_dealloc(tmem_base, 512);
}

}  // namespace gf

using namespace gf;

// ---------------------------------------------------------------------------------------------- host side
namespace {
int fail_if(cudaError_t e) { return e == cudaSuccess ? 0 : gf::fail_cuda(e, "cudaFuncSetAttribute"); }
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// fp16 matrix [rows][K] row-major; box = 128 rows x 64 halves (128 bytes), 128-byte swizzle
int make_map(CUtensorMap *map, void *base, uint64_t rows, uint64_t K) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        GF_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
        GF_REQUIRE(p != nullptr && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled is not available in this driver");
        fn = (EncodeTiledFn)p;
    }
    const cuuint64_t dims[2] = {K, rows};
    const cuuint64_t strides[1] = {K * 2};
    const cuuint32_t box[2] = {FG_BK, FG_BM};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    GF_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed: " + std::to_string((int)r));
    return 0;
}
}  // namespace

struct glmflash_fast_experts {
    glmflash_config cfg;
    __half *xg = nullptr, *xu = nullptr, *xd = nullptr;     // grouped rows
    float *out = nullptr;                                   // pair rows
    int *plan = nullptr, *src_pair = nullptr, *row_expert = nullptr, *status = nullptr;
    CUtensorMap map_xg, map_xu, map_xd;
    int sms = 0;
    int phases = 15;                                        // profiling aid: 1 plan, 2 rotation, 4 gate/up, 8 down
};

extern "C" int glmflash_fast_experts_new(const glmflash_config *cfg, size_t cfg_bytes, glmflash_fast_experts **out) {
    GF_REQUIRE(out != nullptr, "out is null");
    *out = nullptr;
    if (check_config(cfg, cfg_bytes, 8192)) return -1;       // upstream: 1..=8192 rows, src/fast_experts.rs:44-47
    GF_REQUIRE(cfg->experts + 1 <= FG_MAXU, "too many experts for the prefill plan");
    glmflash_fast_experts *f = new (std::nothrow) glmflash_fast_experts();
    GF_REQUIRE(f != nullptr, "out of host memory");
    f->cfg = *cfg;
    const size_t H = cfg->hidden, I = cfg->inter, P = (size_t)cfg->max_rows * cfg->slots;
    auto alloc = [&](void **p, size_t bytes) -> int {
        GF_CUDA(cudaMalloc(p, bytes));
        GF_CUDA(cudaMemset(*p, 0, bytes));
        return 0;
    };
    int dev = 0;
    cudaDeviceProp prop;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaGetDeviceProperties(&prop, dev) != cudaSuccess) {
        delete f;
        return fail("cannot query the CUDA device");
    }
    f->sms = prop.multiProcessorCount;
    if (prop.major != 10) {
        delete f;
        return fail("the prefill path needs an sm_100 GPU (tcgen05 / tensor memory)");
    }
    if (alloc((void **)&f->xg, P * H * 2) || alloc((void **)&f->xu, P * H * 2) || alloc((void **)&f->xd, P * I * 2) ||
        alloc((void **)&f->out, P * H * 4) || alloc((void **)&f->plan, PLAN_INTS * 4) || alloc((void **)&f->src_pair, P * 4) ||
        alloc((void **)&f->row_expert, P * 4) || alloc((void **)&f->status, 16) || make_map(&f->map_xg, f->xg, P, H) ||
        make_map(&f->map_xu, f->xu, P, H) || make_map(&f->map_xd, f->xd, P, I) ||
        fail_if(cudaFuncSetAttribute(fast_gemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FgCfg<2>::SMEM)) ||
        fail_if(cudaFuncSetAttribute(fast_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FgCfg<1>::SMEM))) {
        glmflash_fast_experts_free(f);
        return -1;
    }
    *out = f;
    return 0;
}

extern "C" void glmflash_fast_experts_free(glmflash_fast_experts *f) {
    if (!f) return;
    cudaFree(f->xg); cudaFree(f->xu); cudaFree(f->xd); cudaFree(f->out); cudaFree(f->plan); cudaFree(f->src_pair);
    cudaFree(f->row_expert); cudaFree(f->status);
    delete f;
}

extern "C" int glmflash_fast_experts_run(glmflash_fast_experts *f, void *stream, const glmflash_weights *w, const void *input,
                                         int x_stride, const int32_t *picks, const int32_t *ids, const int32_t *count,
                                         const int32_t *members, int rows, int maxm, int shared_x) {
    GF_REQUIRE(f && w && input && picks && ids && count && members, "null argument");
    const glmflash_config &c = f->cfg;
    GF_REQUIRE(rows > 0 && rows <= c.max_rows && maxm >= rows && maxm <= c.max_rows, "expert rows/member stride outside scratch");
    GF_REQUIRE(x_stride >= c.hidden && x_stride % 4 == 0, "x_stride must be >= hidden and a multiple of 4");
    GF_REQUIRE(((uintptr_t)w->gt | (uintptr_t)w->ut | (uintptr_t)w->dt) % 16 == 0, "trellis tensors must be 16-byte aligned");
    GF_REQUIRE(((uintptr_t)input | (uintptr_t)w->suh_g | (uintptr_t)w->suh_u) % 8 == 0, "input and scale vectors must be 8-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    const int H = c.hidden, I = c.inter;
    const long P = (long)rows * c.slots;
    if (f->phases & 1)
        fast_plan_kernel<<<c.experts + 1, FG_MAXU, 0, s>>>(ids, count, members, maxm, c.slots, c.experts, c.shared_exl3, c.expert_lo,
                                              c.expert_hi, c.shared_row_lo, c.shared_row_hi, f->plan, f->src_pair, f->row_expert);
    GF_CUDA(cudaGetLastError());
    const int mats = shared_x ? 1 : 2;
    if (f->phases & 2)
        fast_rot_kernel<<<(unsigned)std::min<long>(P, 148L * 32), 256, 0, s>>>((const __nv_bfloat16 *)input, x_stride, f->plan, f->src_pair,
                                                              f->row_expert, (const __half *)w->suh_g, (const __half *)w->suh_u,
                                                              f->xg, f->xu, H, c.slots, mats);
    GF_CUDA(cudaGetLastError());
    FastGemmArgs a{};
    a.ids = ids; a.plan = f->plan; a.src_pair = f->src_pair; a.status = f->status; a.limit = c.limit;
    a.T0 = w->gt; a.T1 = w->ut; a.sv0 = (const __half *)w->svh_g; a.sv1 = (const __half *)w->svh_u; a.sd = (const __half *)w->suh_d;
    a.xd = f->xd; a.y = nullptr; a.K = H; a.N = I; a.shared_x = shared_x ? 1 : 0;
    if (f->phases & 4) fast_gemm_kernel<2><<<f->sms, FG_THREADS, FgCfg<2>::SMEM, s>>>(f->map_xg, f->map_xu, a);
    GF_CUDA(cudaGetLastError());
    a.T0 = w->dt; a.T1 = w->dt; a.sv0 = (const __half *)w->svh_d; a.sv1 = nullptr; a.sd = nullptr;
    a.xd = nullptr; a.y = f->out; a.K = I; a.N = H; a.shared_x = 1;
    if (f->phases & 8) fast_gemm_kernel<1><<<f->sms, FG_THREADS, FgCfg<1>::SMEM, s>>>(f->map_xd, f->map_xd, a);
    GF_CUDA(cudaGetLastError());
    return 0;
}

extern "C" int glmflash_fast_experts_set_phases(glmflash_fast_experts *f, int mask) {
    GF_REQUIRE(f != nullptr, "null argument");
    f->phases = mask;
    return 0;
}
extern "C" float *glmflash_fast_experts_output(const glmflash_fast_experts *f) { return f ? f->out : nullptr; }
extern "C" const uint16_t *glmflash_fast_experts_xd(const glmflash_fast_experts *f) { return f ? (const uint16_t *)f->xd : nullptr; }
extern "C" const int32_t *glmflash_fast_experts_row_pairs(const glmflash_fast_experts *f) { return f ? f->src_pair : nullptr; }
extern "C" const int32_t *glmflash_fast_experts_plan(const glmflash_fast_experts *f) { return f ? f->plan : nullptr; }
extern "C" const int32_t *glmflash_fast_experts_status(const glmflash_fast_experts *f) { return f ? f->status : nullptr; }
extern "C" int glmflash_fast_experts_clear_status(glmflash_fast_experts *f, void *stream) {
    GF_REQUIRE(f != nullptr, "null argument");
    GF_CUDA(cudaMemsetAsync(f->status, 0, 4, (cudaStream_t)stream));
    return 0;
}
