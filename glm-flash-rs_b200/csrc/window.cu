// The whole MoE layer for a window of 1..16 rows (decode and speculative verify) in ONE launch, sm_100a.
//
// Upstream runs five kernels per window (rot_in, grouped gate/up, gateup_epilogue, grouped down, down_epilogue:
// src/experts.rs:447-563, native/exl3.cu:224-330) after a grouping kernel and before a combine kernel
// (src/moe.rs:66-182), and an all-gather + ordered sum across ranks behind that (src/model.rs:485-496).  At one
// token the layer streams 24 MB of packed words, about four microseconds of HBM time, so kernel boundaries and
// round trips through memory, not bytes, decide how long it takes.  Here one persistent CTA per SM does all of it as
// a dataflow over three kinds of work items:
//
//   G  (expert, matrix, 128-k split, 256-column block) of the gate / up projections,
//   D  (expert, 128-k split, 256-column block) of the down projection,
//   F  (row, 128-column block) of the layer output.
//
//   * grouping: every CTA derives the distinct experts of the window and their members from the routing table
//     itself (80 entries at most), in shared memory: same result as native/grouping.cu, no launch;
//   * a CTA is two teams of eight compute warps and one service warp (more teams would leave the K loop fewer than
//     the 96 registers it needs to stay free of spills; measured).  Each kind's items are cut into equal
//     contiguous ranges, one per team, teams numbered SM-major, so that every SM decodes the same number of bytes
//     (the decode is instruction-issue bound) and the items of a team that share (expert, matrix, split) -- a run --
//     share one staging of the members' activations;
//   * weight stream: a G or D item is 8 rows of 2 KB of packed trellis words; a team owns four 16-KB buffers.  The
//     service warp requests the copies (TMA bulk copies, cp.async.bulk, completion counted on mbarriers): the first
//     four items before anything else happens, item q + 4 when the compute warps have left item q (they count
//     themselves out on an mbarrier) -- the compute warps never wait for the copy engine to accept a request;
//   * math: the decode GEMV's inner loop (gemv.cuh): a lane reads 16 bytes = 32 weights, cuts the 16-bit trellis
//     states with funnel shifts, decodes the codebook in registers bit-exactly, and feeds mma.m16n8k16 with the
//     weights as A over a doubled K and the members (<= 8 per set, two sets for 9..16) as N; a warp owns two
//     n-tiles that share the B operands; fp32 accumulation.  The loop is call-free and spill-free: everything else
//     a compute warp does lives in out-of-line functions, and the loop state is one counter and one packed word;
//   * an item leaves its split's partial in a fixed place in global scratch (L2); the service warp then raises the
//     item's flag word to the launch's epoch with a release store (the fence behind it is a round trip to the L2:
//     paid by the service warp, not by a warp that decodes).  Nothing is counted and nothing is reset: a consumer
//     polls (bounded, acquire loads) the flag words of exactly the partials it reads;
//   * a G run rotates the members' input block itself (upstream rot_in_kernel); a D run waits for the 2 x H/128 gate
//     and up partials of its 128 k, adds them (groups of eight splits in ascending order, then the groups in
//     ascending order: one round trip to the L2) and runs the gate/up epilogue (Hadamard, scales, limited SwiGLU with
//     upstream's rounding points, down-input scale, Hadamard) straight into its staged operands; an F item waits for
//     the down partials of the row's pairs, finishes each pair (Hadamard, output scale -> Y) and adds the pairs in
//     ascending slot order (the combine).  Every sum has an order fixed by the shape, so no value depends on timing
//     and a row has the bits of its 1-row call;
//   * expert parallel: the F item stores its block into every peer's receive slot over NVLink (plain peer stores, no
//     multicast) and raises a per-block flag; when a team has finished its items it waits (bounded) for the peers'
//     blocks it owes and adds the slots in rank order (the reference's fixed-order sum).
// No grid-wide barrier, no atomics on the data path, every wait bounded with a status word.
#include <stddef.h>

#include <algorithm>

#include "gemv.cuh"
#include "owners.cuh"

namespace gf {

#ifndef WIN_TEAMS_N
#define WIN_TEAMS_N 2
#endif
constexpr int WIN_TEAMS = WIN_TEAMS_N;
constexpr int WIN_CW = 8;                                     // compute warps of a team
constexpr int WIN_TEAM_WARPS = WIN_CW + 1;                    // + the service warp: copy requests, flag publication
constexpr int WIN_THREADS = WIN_TEAMS * WIN_TEAM_WARPS * 32;
constexpr int WIN_KTI = 8;                                    // k-tiles of an item
constexpr int WIN_KC = WIN_KTI * 16;                          // 128 k: one Hadamard block
constexpr int WIN_NG = WIN_KTI / 4;                           // copy barriers of a buffer (four k-tiles each)
constexpr int WIN_COLS = 256;                                 // columns of an item: 16 n-tiles, two per warp
constexpr int WIN_WROW = WIN_COLS * 8 + 32;                   // bytes per staged row (2 KB + 32 B: conflict-free LDS.128)
constexpr int WIN_WBUF = WIN_KTI * WIN_WROW;                  // bytes of a weight buffer
#ifndef WIN_NBUF_N
#define WIN_NBUF_N 4
#endif
constexpr int WIN_NBUF = WIN_NBUF_N;                          // weight buffers of a team
constexpr int WIN_ACT = 8 * (WIN_KC + 8) * 4;                 // staged activations: 8 x (128 + 8) dwords = 16 x (64 + 4)
constexpr int WIN_SCR = 16 * 512;                             // split-sum scratch: 16 partial rows of 128 floats
constexpr int WIN_TEAM_BYTES = WIN_NBUF * WIN_WBUF + WIN_ACT + WIN_SCR;
constexpr int WIN_BARS = WIN_NBUF * (WIN_NG + 1);             // per team: copy barriers and one "consumed" barrier per buffer
constexpr int WIN_UMAX = 160;                                 // distinct experts of a window the tables hold
constexpr int WIN_QMAX = 32;                                  // deferred exchange blocks a team can hold (its F items)
constexpr int WIN_MAXSPLIT = 32;                              // splits per projection the split-sum scratch handles (K <= 4096)
constexpr size_t WIN_SMEM = (size_t)WIN_TEAMS * WIN_TEAM_BYTES + WIN_TEAMS * WIN_BARS * 8;
constexpr uint32_t WIN_POLLS = 2000000u;                      // bound of every spin in the kernel (a fraction of a second)

// WIN_TRACE (timing experiments only): lane 0 of compute warp 0 (WIN_STAMP) and of the service warp (WIN_STAMP_S) of every
// team stamp the global nanosecond timer into a buffer registered with glmflash_win_trace_set(): [CTA][team][64] int64.
#ifdef WIN_TRACE
static __device__ long long *g_win_trace = nullptr;
#define WIN_STAMP_(slot, cond)                                                                                         \
    do {                                                                                                               \
        if ((cond) && g_win_trace && (slot) >= 0 && (slot) < 64) {                                                     \
            long long t_;                                                                                              \
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_));                                                      \
            g_win_trace[((size_t)blockIdx.x * WIN_TEAMS + threadIdx.x / (WIN_TEAM_WARPS * 32)) * 64 + (slot)] = t_;    \
        }                                                                                                              \
    } while (0)
#define WIN_STAMP(slot) WIN_STAMP_((slot) < 32 ? (slot) : -1, threadIdx.x % (WIN_TEAM_WARPS * 32) == 0)
#define WIN_STAMP_S(slot) WIN_STAMP_(slot, (threadIdx.x & 31) == 0)
#else
#define WIN_STAMP(slot) do { } while (0)
#define WIN_STAMP_S(slot) do { } while (0)
#endif

struct WinArgs {
    const __nv_bfloat16 *x;
    const int *picks;
    const float *route_w;
    const uint32_t *gt, *ut, *dt;
    const __half *suh_g, *suh_u, *suh_d, *svh_g, *svh_u, *svh_d;
    __half *xd;
    float *z1, *z2, *y, *out;
    unsigned *sync;
    int *status;
    int rows, slots, H, I, E, e_lo, e_hi, shared_exl3, x_stride;
    float limit;
    WinPeers peers;                                           // world <= 1: single GPU
};

// sync words: [0] epoch, [1] finished output blocks, then the flag words: one per G item of every expert
// [E1][I/256][2 * H/128] and one per D item [E1][H/256][I/128], each block of words padded to a multiple of 32.
__device__ __host__ __forceinline__ int win_pad32(int n) { return (n + 31) & ~31; }
__device__ __forceinline__ unsigned *win_fg(const WinArgs &a, int e, int nb2) {
    return a.sync + 32 + ((size_t)e * (a.I >> 8) + nb2) * win_pad32(2 * (a.H >> 7));
}
__device__ __forceinline__ unsigned *win_fd(const WinArgs &a, int e, int nb2) {
    return a.sync + 32 + (size_t)(a.E + 1) * (a.I >> 8) * win_pad32(2 * (a.H >> 7)) + ((size_t)e * (a.H >> 8) + nb2) * win_pad32(a.I >> 7);
}
inline size_t win_sync_words(int E, int H, int I) {
    return 32 + (size_t)(E + 1) * ((size_t)(I >> 8) * win_pad32(2 * (H >> 7)) + (size_t)(H >> 8) * win_pad32(I >> 7));
}

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned *p, unsigned v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned atom_add_acq_rel_gpu(unsigned *p, unsigned v) {
    unsigned old;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u32(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// mma without `volatile`: the scheduler may move the decode of the next operands across it.
__device__ __forceinline__ void win_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Barrier of a team's compute warps (the service warp does not take part).
__device__ __forceinline__ void team_bar(int team) { asm volatile("bar.sync %0, 256;" ::"r"(team + 1) : "memory"); }
// A value the compiler must treat as new: keeps it from hoisting per-item arithmetic out of the item loop (where it
// would occupy registers across the K loop).
__device__ __forceinline__ int win_opaque(int x) {
    asm volatile("" : "+r"(x));
    return x;
}
// Position of a thread: team, and warp within the team (WIN_CW = the service warp).
__device__ __forceinline__ int win_team() { return (threadIdx.x >> 5) / WIN_TEAM_WARPS; }
__device__ __forceinline__ int win_warp() { return (threadIdx.x >> 5) % WIN_TEAM_WARPS; }

// Bounded wait on a TMA barrier; the waiting thread may sleep inside the instruction, so it takes no issue slots from
// the warps that decode.
__device__ __forceinline__ bool win_mbar_wait(uint64_t *bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    for (uint32_t i = 0; i < WIN_POLLS; ++i)
        if (mbar_try_wait_hint(bar, parity, 500u)) return true;
    return false;
}
// The same with a short bound (tens of milliseconds), for the way out after a give-up.
__device__ __forceinline__ void win_mbar_drain(uint64_t *bar, uint32_t parity) {
    for (uint32_t i = 0; i < 40000u; ++i)
        if (mbar_try_wait_hint(bar, parity, 500u)) return;
}
// Bounded wait of a whole warp until the n flag words from f on all hold `want`.
__device__ __forceinline__ bool win_wait_flags(const unsigned *f, int n, unsigned want) {
    const int lane = threadIdx.x & 31;
    for (int n0 = 0; n0 < n; n0 += 32) {
        bool ok = false;
        for (uint32_t i = 0; i < WIN_POLLS && !ok; ++i) {
            const bool mine = n0 + lane >= n || ld_acquire_gpu(f + n0 + lane) == want;
            ok = __all_sync(0xffffffffu, mine);
            if (!ok && i > 16) __nanosleep(64);
        }
        if (!ok) return false;
    }
    return true;
}

// ---- items.  G: index = ((u * 2 + mat) * SKg + split) * NB2g + nb2;  D: (u * SKd + split) * NB2d + nb2;  F: row * NBd + nb.
// An item is carried as one packed word (kind 2 bits | u 9 | mat 1 | split 8 | nb2 8) and advanced without divisions.
struct WinShape {
    int NB2g, SKg, NB2d, SKd, n_g, n_d, n_f;
};
__device__ __forceinline__ WinShape win_shape(int H, int I, int U, int rows) {
    WinShape s;
    s.NB2g = I >> 8; s.SKg = H / WIN_KC; s.NB2d = H >> 8; s.SKd = I / WIN_KC;
    s.n_g = U * 2 * s.SKg * s.NB2g; s.n_d = U * s.SKd * s.NB2d; s.n_f = rows * 2 * s.NB2d;
    return s;
}
struct WinItem {
    uint32_t w;
    __device__ __forceinline__ int kind() const { return (int)(w >> 26); }
    __device__ __forceinline__ int u() const { return (int)((w >> 17) & 511u); }       // F: the row
    __device__ __forceinline__ int mat() const { return (int)((w >> 16) & 1u); }
    __device__ __forceinline__ int split() const { return (int)((w >> 8) & 255u); }
    __device__ __forceinline__ int nb2() const { return (int)(w & 255u); }             // F: the 128-column block
    __device__ __forceinline__ uint32_t run_key() const { return w >> 8; }
};
__device__ __forceinline__ WinItem win_pack(int kind, int u, int mat, int split, int nb2) {
    WinItem it;
    it.w = ((uint32_t)kind << 26) | ((uint32_t)u << 17) | ((uint32_t)mat << 16) | ((uint32_t)split << 8) | (uint32_t)nb2;
    return it;
}
__device__ __forceinline__ WinItem win_item_at(const WinShape &s, int kind, int i) {   // by division: three times per team
    if (kind == 0) {
        const int nb2 = i % s.NB2g;
        int r = i / s.NB2g;
        const int split = r % s.SKg;
        r /= s.SKg;
        return win_pack(0, r >> 1, r & 1, split, nb2);
    }
    if (kind == 1) {
        const int nb2 = i % s.NB2d, r = i / s.NB2d;
        return win_pack(1, r / s.SKd, 0, r % s.SKd, nb2);
    }
    return win_pack(2, i / (2 * s.NB2d), 0, 0, i % (2 * s.NB2d));
}
__device__ __forceinline__ WinItem win_item_next(const WinShape &s, WinItem it) {      // the item after `it` of the same kind
    const int kind = it.kind();
    int u = it.u(), mat = it.mat(), split = it.split(), nb2 = it.nb2() + 1;
    const int NB = kind == 0 ? s.NB2g : kind == 1 ? s.NB2d : 2 * s.NB2d;
    if (nb2 == NB) {
        nb2 = 0;
        if (kind == 2) ++u;
        else {
            ++split;
            if (split == (kind == 0 ? s.SKg : s.SKd)) {
                split = 0;
                if (kind == 0 && mat == 0) mat = 1;
                else { mat = 0; ++u; }
            }
        }
    }
    return win_pack(kind, u, mat, split, nb2);
}

// Tables of a CTA (static shared memory): the window's grouping and the teams' plans.
struct __align__(16) WinShared {
    float up[WIN_TEAMS][4][128];                              // gate/up epilogue: the up values of a warp pair's block (float4 access)
    int picks[512];
    int ids[WIN_UMAX], cnt[WIN_UMAX];
    unsigned short mem[WIN_UMAX][16];                         // members (pair indices) of distinct expert u, ascending rows
    uint32_t used[32], rowlive[16];                           // experts computed here (bitmap); per row: slots computed here
    int base[33];
    int U;
    int abort[WIN_TEAMS], qn[WIN_TEAMS];
    unsigned short queue[WIN_TEAMS][WIN_QMAX];                // expert parallel: blocks pushed by the team, to be summed
    // The plan of a team, written once at set-up.  The compute loop reads it from here at every item instead of keeping
    // it in registers: the K loop needs nearly every register a thread has, and a value that stayed live across it
    // would be spilled to local memory, which at this occupancy misses the L1.
    struct Plan {
        int g0, d0, f0, ngl, nw, nloc;
    } plan[WIN_TEAMS];
    unsigned epoch, xepoch;
};
static_assert(offsetof(WinShared, up) % 16 == 0, "float4 access");

// Item q of a team's sequence (its G items, then its D items, then its F items), from item q - 1.
__device__ __forceinline__ WinItem win_local_next(const WinShape &s, const WinShared::Plan &pl, int q, WinItem prev) {
    if (q == 0) return pl.ngl > 0 ? win_item_at(s, 0, pl.g0) : pl.nw > 0 ? win_item_at(s, 1, pl.d0) : win_item_at(s, 2, pl.f0);
    if (q == pl.ngl) return pl.nw > pl.ngl ? win_item_at(s, 1, pl.d0) : win_item_at(s, 2, pl.f0);
    if (q == pl.nw) return win_item_at(s, 2, pl.f0);
    return win_item_next(s, prev);
}

// One lane: the last finished output block of the launch advances the epochs (every CTA read them at its start).
__device__ __forceinline__ void win_finish_count(const WinArgs &a, unsigned epoch, unsigned xepoch) {
    const unsigned total = (unsigned)(a.rows * (a.H >> 7));
    if (atom_add_acq_rel_gpu(a.sync + 1, 1u) == total - 1u) {
        a.sync[1] = 0u;
        if (a.peers.world > 1) *a.peers.epoch = xepoch;
        __threadfence();
        a.sync[0] = epoch;
    }
}

// The final step of an output block (row, 128 columns), by a whole warp; v: the lane's four columns.  Single GPU:
// store.  Expert parallel: store into slot `rank` of every rank's receive area (plain peer stores over NVLink), raise
// the block's flag there, and remember the block: the team adds the ranks' slots when its items are done.
__device__ __forceinline__ void win_block_out(const WinArgs &a, WinShared &sh, int team, int row, int nb, float4 v, unsigned epoch,
                                              unsigned xepoch) {
    const int lane = threadIdx.x & 31, H = a.H, NBd = H >> 7;
    const size_t off = (size_t)row * H + nb * 128 + 4 * lane;
    if (a.peers.world <= 1) {
        __stcg(reinterpret_cast<float4 *>(a.out + off), v);
        __syncwarp();
        if (lane == 0) win_finish_count(a, epoch, xepoch);
        return;
    }
    const unsigned par = xepoch & 1u;
    const size_t slot = (size_t)a.peers.max_rows * H;
    for (int k = 0; k < a.peers.world; ++k)
        *reinterpret_cast<float4 *>(a.peers.recv[k] + ((size_t)par * a.peers.world + a.peers.rank) * slot + off) = v;
    __threadfence_system();
    __syncwarp();
    if (lane < a.peers.world)
        st_release_sys_u32(a.peers.flags[lane] + (((size_t)par * a.peers.world + a.peers.rank) * a.peers.max_rows + row) * NBd + nb, xepoch);
    if (lane == 0) {
        const int q = atomicAdd(&sh.qn[team], 1);
        if (q < WIN_QMAX) sh.queue[team][q] = (unsigned short)(row * NBd + nb);
    }
}

// Sum of up to eight consecutive splits' partials (planes zs0 ..) of pair p, columns n0..n0+3, in ascending order: all
// loads of the group are in flight together.
__device__ __forceinline__ float4 win_sum_group(const float *Z, int zs0, int n, size_t P, int p, int N, int n0) {
    const float *zp = Z + ((size_t)zs0 * P + p) * N + n0;
    const size_t step = P * N;
    float4 q[8];
#pragma unroll
    for (int s = 0; s < 8; ++s)
        if (s < n) q[s] = __ldcg(reinterpret_cast<const float4 *>(zp + (size_t)s * step));
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < 8; ++s)
        if (s < n) { v.x += q[s].x; v.y += q[s].y; v.z += q[s].z; v.w += q[s].w; }
    return v;
}
__device__ __forceinline__ void win_scale4(const __half *vec, float (&o)[4]) {
    const uint2 raw = __ldg(reinterpret_cast<const uint2 *>(vec));
    const __half2 s01 = *reinterpret_cast<const __half2 *>(&raw.x), s23 = *reinterpret_cast<const __half2 *>(&raw.y);
    o[0] = __low2float(s01); o[1] = __high2float(s01); o[2] = __low2float(s23); o[3] = __high2float(s23);
}

// Expert parallel: the blocks this team pushed.  Wait (bounded) for every rank's copy, add the slots in rank order.
__device__ __noinline__ void win_exchange_sum(const WinArgs &a, WinShared &sh, int team, unsigned epoch, unsigned xepoch) {
    const int warp = win_warp(), lane = threadIdx.x & 31;
    const int H = a.H, NBd = H >> 7;
    const int qn = min(sh.qn[team], WIN_QMAX);
    const unsigned par = xepoch & 1u;
    const size_t slot = (size_t)a.peers.max_rows * H;
    for (int q = warp; q < qn; q += WIN_CW) {
        const int row = sh.queue[team][q] / NBd, nb = sh.queue[team][q] % NBd;
        bool ok = true;
        if (lane < a.peers.world) {
            const unsigned *f = a.peers.flags[a.peers.rank] + (((size_t)par * a.peers.world + lane) * a.peers.max_rows + row) * NBd + nb;
            ok = false;
            for (uint32_t t = 0; t < a.peers.wait_polls; ++t) {
                if (ld_acquire_sys_u32(f) == xepoch) { ok = true; break; }
                if (t > 64) __nanosleep(100);
                if ((t & 1023u) == 1023u && *reinterpret_cast<volatile int *>(a.peers.status) == GF_STATUS_PEER_TIMEOUT) break;
            }
            if (!ok) atomicExch(a.peers.status, GF_STATUS_PEER_TIMEOUT);
        }
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            const size_t off = (size_t)row * H + nb * 128 + 4 * lane;
            const float *src = a.peers.recv[a.peers.rank] + (size_t)par * a.peers.world * slot + off;
            float4 sum = __ldcg(reinterpret_cast<const float4 *>(src));
            for (int k = 1; k < a.peers.world; ++k) {
                const float4 v = __ldcg(reinterpret_cast<const float4 *>(src + (size_t)k * slot));
                sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
            }
            __stcg(reinterpret_cast<float4 *>(a.out + off), sum);
        }
        __syncwarp();
        if (lane == 0) win_finish_count(a, epoch, xepoch);
    }
}

// Staged activations of a team: one row of AST dwords per member.  Two member sets (9..16 members): fp16 in natural k
// order (AST = KC / 2 + 4 keeps the 16-byte reads of the K loop free of bank conflicts), the (x_k, 0) operand pairs are
// cut in the K loop.  One set: ready-made (x_k, 0) dword pairs in mma order: the pair of local
// k = 64 g + 16 T + 8 h + 2 t + b sits at dword g*64 + (2t + h)*8 + 2T + b.
template <int SETS>
struct WinStage {
    static constexpr bool PACKED = SETS == 2;
    static constexpr int AST = PACKED ? (WIN_KC >> 1) + 4 : WIN_KC + 8;
    static __device__ __forceinline__ int pos(int kl) {
        const int g = kl >> 6, TT = (kl >> 4) & 3, h = (kl >> 3) & 1, t = (kl >> 1) & 3;
        return g * 64 + (2 * t + h) * 8 + 2 * TT;
    }
    static __device__ __forceinline__ void put4(uint32_t *row, int kl, uint32_t w01, uint32_t w23) {   // k = kl .. kl + 3
        if (PACKED) {
            *reinterpret_cast<uint2 *>(row + (kl >> 1)) = make_uint2(w01, w23);
        } else {
            *reinterpret_cast<uint2 *>(row + pos(kl)) = make_uint2(w01 & 0xffffu, w01 >> 16);
            *reinterpret_cast<uint2 *>(row + pos(kl + 2)) = make_uint2(w23 & 0xffffu, w23 >> 16);
        }
    }
};

// Staging of a G run: fp16(H(x * suh) / sqrt 128) of the run's 128-block, one warp per member (upstream
// rot_in_kernel, native/exl3.cu:224-241: same butterflies, same rounding).
template <int SETS>
__device__ __noinline__ void win_stage_rotate(const WinArgs &a, uint32_t *act, const unsigned short *mem, int nmem, int e, int mat, int k0) {
    using St = WinStage<SETS>;
    const int warp = win_warp(), lane = threadIdx.x & 31;
    for (int m = warp; m < nmem; m += WIN_CW) {
        const int row = mem[m] / a.slots;
        const uint2 xv = __ldcg(reinterpret_cast<const uint2 *>(a.x + (size_t)row * a.x_stride + k0 + 4 * lane));
        const uint2 sv = __ldg(reinterpret_cast<const uint2 *>((mat ? a.suh_u : a.suh_g) + (size_t)e * a.H + k0 + 4 * lane));
        const __nv_bfloat162 x01 = *reinterpret_cast<const __nv_bfloat162 *>(&xv.x), x23 = *reinterpret_cast<const __nv_bfloat162 *>(&xv.y);
        const __half2 s01 = *reinterpret_cast<const __half2 *>(&sv.x), s23 = *reinterpret_cast<const __half2 *>(&sv.y);
        float v[4] = {__bfloat162float(x01.x) * __low2float(s01), __bfloat162float(x01.y) * __high2float(s01),
                      __bfloat162float(x23.x) * __low2float(s23), __bfloat162float(x23.y) * __high2float(s23)};
        fwht128(v, lane);
        const __half2 r01 = __halves2half2(__float2half_rn(v[0] * HAD_SCALE), __float2half_rn(v[1] * HAD_SCALE));
        const __half2 r23 = __halves2half2(__float2half_rn(v[2] * HAD_SCALE), __float2half_rn(v[3] * HAD_SCALE));
        St::put4(act + (size_t)m * St::AST, 4 * lane, *reinterpret_cast<const uint32_t *>(&r01), *reinterpret_cast<const uint32_t *>(&r23));
    }
}

// Staging of a D run = the gate/up epilogue of its 128 columns of the intermediate (upstream gateup_epilogue_kernel,
// native/exl3.cu:260-296), four members per pass:
//   A. a warp adds a group of up to eight consecutive splits of (member, matrix) with all loads in flight together and
//      leaves the group's sum in shared memory;
//   B. a warp pair per member: each adds its matrix's groups in ascending order, Hadamard, scales; the odd warp clamps
//      the up values and hands them over through shared memory, the even warp does gate, limited SwiGLU with upstream's
//      rounding points, the down-input scale, the second Hadamard, and writes fp16 to the staged operands (and to xd, for
//      the probes).
template <int SETS>
__device__ __noinline__ void win_stage_swiglu(const WinArgs &a, WinShared &sh, uint32_t *act, float *scr, const unsigned short *mem,
                                              int nmem, int e, int split, int team) {
    using St = WinStage<SETS>;
    const int warp = win_warp(), lane = threadIdx.x & 31;
    const int I = a.I, SKg = a.H / WIN_KC, n0 = split * WIN_KC + 4 * lane;
    const int NGR = (SKg + 7) >> 3;                            // groups per matrix (<= 4: scratch rows = 4 members x 2 x NGR <= 32 ... see below)
    const size_t P = (size_t)a.rows * a.slots;
    // members per pass: the scratch holds 16 group sums = mp members x 2 matrices x NGR groups
    const int mp = NGR <= 2 ? 4 : NGR <= 4 ? 2 : 1;
    for (int m0 = 0; m0 < nmem; m0 += mp) {
        const int mc = min(mp, nmem - m0), tasks = mc * 2 * NGR;
        for (int t = warp; t < tasks; t += WIN_CW) {          // A
            const int g = t % NGR, mm = t / NGR, mat = mm & 1, ml = mm >> 1;
            const float4 v = win_sum_group(a.z1, mat * SKg + g * 8, min(8, SKg - g * 8), P, mem[m0 + ml], I, n0);
            *reinterpret_cast<float4 *>(scr + (size_t)t * 128 + 4 * lane) = v;
        }
        team_bar(team);
        const int pair = warp >> 1, role = warp & 1;           // B
        const bool on = pair < mc;
        float sg[4];
        if (on) {
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            for (int g = 0; g < NGR; ++g) {
                const float4 q = *reinterpret_cast<const float4 *>(scr + (size_t)((pair * 2 + role) * NGR + g) * 128 + 4 * lane);
                v[0] += q.x; v[1] += q.y; v[2] += q.z; v[3] += q.w;
            }
            fwht128(v, lane);
            float sc[4];
            win_scale4((role ? a.svh_u : a.svh_g) + (size_t)e * I + n0, sc);
            if (role == 1) {
                float4 uu;
                uu.x = fminf(fmaxf(bf16r(v[0] * HAD_SCALE * sc[0]), -a.limit), a.limit);
                uu.y = fminf(fmaxf(bf16r(v[1] * HAD_SCALE * sc[1]), -a.limit), a.limit);
                uu.z = fminf(fmaxf(bf16r(v[2] * HAD_SCALE * sc[2]), -a.limit), a.limit);
                uu.w = fminf(fmaxf(bf16r(v[3] * HAD_SCALE * sc[3]), -a.limit), a.limit);
                *reinterpret_cast<float4 *>(&sh.up[team][pair][4 * lane]) = uu;
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float gg = fminf(bf16r(v[q] * HAD_SCALE * sc[q]), a.limit);
                    sg[q] = bf16r(gg / (1.f + expf(-gg)));
                }
            }
        }
        team_bar(team);                                        // up values are there; the scratch may be written again
        if (on && role == 0) {
            const int m = m0 + pair, p = mem[m];
            const float4 uu = *reinterpret_cast<const float4 *>(&sh.up[team][pair][4 * lane]);
            float sd_[4], o[4];
            win_scale4(a.suh_d + (size_t)e * I + n0, sd_);
            o[0] = bf16r(sg[0] * uu.x) * sd_[0];
            o[1] = bf16r(sg[1] * uu.y) * sd_[1];
            o[2] = bf16r(sg[2] * uu.z) * sd_[2];
            o[3] = bf16r(sg[3] * uu.w) * sd_[3];
            fwht128(o, lane);
            const __half2 h01 = __halves2half2(__float2half_rn(o[0] * HAD_SCALE), __float2half_rn(o[1] * HAD_SCALE));
            const __half2 h23 = __halves2half2(__float2half_rn(o[2] * HAD_SCALE), __float2half_rn(o[3] * HAD_SCALE));
            const uint32_t w01 = *reinterpret_cast<const uint32_t *>(&h01), w23 = *reinterpret_cast<const uint32_t *>(&h23);
            St::put4(act + (size_t)m * St::AST, 4 * lane, w01, w23);
            __stcg(reinterpret_cast<uint2 *>(a.xd + (size_t)p * I + n0), make_uint2(w01, w23));
        }
        if (m0 + mp < nmem) team_bar(team);                    // up may be written again
    }
}

// An F item: output block (row, 128 columns nb), eight slots per pass:
//   A. a warp waits for the down partials of a slot's pair (when the pair is computed here) and adds a group of up to
//      eight consecutive splits; B. a warp per slot adds the groups in ascending order, Hadamard, output scale -> Y
//      (upstream down_epilogue_kernel, native/exl3.cu:300-321) and leaves the block in shared memory; C. warp 0 adds the
//      pairs in ascending slot order, the shared slot last and unweighted (the combine upstream runs as a separate kernel,
//      src/moe.rs:171-181).
__device__ __noinline__ bool win_finish_block(const WinArgs &a, WinShared &sh, float *fbuf, float *scr, int row, int nb, int team,
                                              unsigned epoch, unsigned xepoch) {
    const int warp = win_warp(), lane = threadIdx.x & 31;
    const int H = a.H, SKd = a.I / WIN_KC, n0 = nb * 128 + 4 * lane;
    const int NGR = (SKd + 7) >> 3, sp = NGR <= 2 ? 8 : NGR <= 4 ? 4 : 2;     // slots per pass (scratch: 16 group sums)
    const size_t P = (size_t)a.rows * a.slots;
    const uint32_t live = sh.rowlive[row];
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < a.slots; s0 += sp) {
        const int sc_ = min(sp, a.slots - s0), tasks = sc_ * NGR;
        bool ok = true;
        for (int t = warp; t < tasks; t += WIN_CW) {          // A
            const int g = t % NGR, s = s0 + t / NGR;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if ((live >> s) & 1u) {
                const int p = row * a.slots + s, e = sh.picks[p];
                ok = win_wait_flags(win_fd(a, e, nb >> 1) + g * 8, min(8, SKd - g * 8), epoch);
                if (ok) v = win_sum_group(a.z2, g * 8, min(8, SKd - g * 8), P, p, H, n0);
            }
            *reinterpret_cast<float4 *>(scr + (size_t)t * 128 + 4 * lane) = v;
        }
        if (!ok && lane == 0) { atomicExch(a.status, GF_STATUS_PEER_TIMEOUT); sh.abort[team] = 1; }
        team_bar(team);
        if (warp < sc_ && ((live >> (s0 + warp)) & 1u)) {     // B
            const int s = s0 + warp, p = row * a.slots + s, e = sh.picks[p];
            float v[4] = {0.f, 0.f, 0.f, 0.f}, sd_[4];
            for (int g = 0; g < NGR; ++g) {
                const float4 q = *reinterpret_cast<const float4 *>(scr + (size_t)(warp * NGR + g) * 128 + 4 * lane);
                v[0] += q.x; v[1] += q.y; v[2] += q.z; v[3] += q.w;
            }
            win_scale4(a.svh_d + (size_t)e * H + n0, sd_);
            fwht128(v, lane);
            float4 o;
            o.x = v[0] * HAD_SCALE * sd_[0];
            o.y = v[1] * HAD_SCALE * sd_[1];
            o.z = v[2] * HAD_SCALE * sd_[2];
            o.w = v[3] * HAD_SCALE * sd_[3];
            __stcg(reinterpret_cast<float4 *>(a.y + (size_t)p * H + n0), o);
            *reinterpret_cast<float4 *>(fbuf + warp * 128 + 4 * lane) = o;
        }
        team_bar(team);
        if (warp == 0) {                                       // C
            for (int w = 0; w < sc_; ++w) {
                if (!((live >> (s0 + w)) & 1u)) continue;
                const float4 yv = *reinterpret_cast<const float4 *>(fbuf + w * 128 + 4 * lane);
                if (s0 + w == a.slots - 1) { sum.x += yv.x; sum.y += yv.y; sum.z += yv.z; sum.w += yv.w; }
                else {
                    const float wgt = __ldg(a.route_w + row * a.slots + s0 + w);
                    sum.x += wgt * yv.x; sum.y += wgt * yv.y; sum.z += wgt * yv.z; sum.w += wgt * yv.w;
                }
            }
        }
        if (s0 + sp < a.slots) team_bar(team);                 // fbuf and the scratch may be written again
    }
    if (sh.abort[team]) return false;
    if (warp == 0) win_block_out(a, sh, team, row, nb, sum, epoch, xepoch);
    return true;
}

// The K loop of a G or D item and the store of this split's partials.  Warp w owns n-tiles w and w + 8 of the 256-column
// block (they share the B operands); zb points at [pair 0][first column of the block] of the split's plane, rows of N
// floats.  Returns false when a copy did not arrive within the bound.
template <int SETS>
__device__ __forceinline__ bool win_kloop(const unsigned char *wbuf, const uint32_t *act, uint64_t *bars, uint32_t par, int nmem,
                                          const unsigned short *mem, float *zb, int N) {
    using St = WinStage<SETS>;
    constexpr bool PACKED = St::PACKED;
    constexpr int AST = St::AST;
    const int warp = win_warp(), lane = threadIdx.x & 31;
    const int G = lane >> 2, T = lane & 3;
    const bool two_sets = SETS == 2 && nmem > 8;
    float acc[2][SETS][4];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int s = 0; s < SETS; ++s)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[n][s][c] = 0.f;
    bool ok = true;
#pragma unroll 1
    for (int g = 0; g < WIN_NG; ++g) {
        // B operands of the group's 8 mma: the 16 activations k = 64 g + 16 T .. + 15 of member G (and 8 + G)
        uint32_t bp[SETS][8];
        uint2 b1[8];
        if (PACKED) {
#pragma unroll
            for (int s = 0; s < SETS; ++s) {
                const uint4 *ar = reinterpret_cast<const uint4 *>(act + (size_t)(s * 8 + G) * AST + g * 32 + 8 * T);
                const uint4 lo = ar[0], hi = ar[1];
                bp[s][0] = lo.x; bp[s][1] = lo.y; bp[s][2] = lo.z; bp[s][3] = lo.w;
                bp[s][4] = hi.x; bp[s][5] = hi.y; bp[s][6] = hi.z; bp[s][7] = hi.w;
            }
        } else {
            const uint32_t *ar = act + (size_t)G * AST + g * 64 + 2 * T;
#pragma unroll
            for (int m = 0; m < 8; ++m) b1[m] = *reinterpret_cast<const uint2 *>(ar + m * 8);
        }
        if (!win_mbar_wait(bars + g, par)) { ok = false; break; }
        const unsigned char *wrow = wbuf + (size_t)(4 * g + T) * WIN_WROW + warp * 128 + G * 16;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const uint4 wv = *reinterpret_cast<const uint4 *>(wrow + n * 1024);
            const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
            const uint32_t before = __shfl_sync(0xffffffffu, wv.w, (lane + 28) & 31);       // word 4G-1 (circular)
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
#ifdef WIN_EXP_NODECODE
                    af[0] = uu[2 * h]; af[1] = uu[2 * h + 1]; af[2] = uu[2 * h] ^ pw; af[3] = uu[2 * h + 1] ^ pw;
                    (void)x0; (void)x1; (void)x2; (void)x3;
#else
                    codeword_pair(uu[2 * h], x0, x1);        // k = 2t + 8h:     columns G, G + 8
                    codeword_pair(uu[2 * h + 1], x2, x3);    // k = 2t + 8h + 1: columns G, G + 8
                    af[0] = weight_dup(x0); af[1] = weight_dup(x1); af[2] = weight_dup(x2); af[3] = weight_dup(x3);
#endif
                    if (!PACKED) {
                        win_mma(acc[n][0], af, b1[2 * t + h].x, b1[2 * t + h].y);
                    } else {
                        const uint32_t bw0 = bp[0][4 * h + t];
                        win_mma(acc[n][0], af, bw0 & 0xffffu, bw0 >> 16);
                    }
                    if (SETS == 2 && two_sets) {
                        const uint32_t bw1 = bp[SETS - 1][4 * h + t];
                        win_mma(acc[n][SETS - 1], af, bw1 & 0xffffu, bw1 >> 16);
                    }
                }
            }
        }
    }
    // accumulator c of (n, s): column G (c < 2) or G + 8 of n-tile w + 8 n, member 8 s + 2 T + (c & 1)
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int s = 0; s < SETS; ++s)
#pragma unroll
            for (int mm = 0; mm < 2; ++mm) {
                const int m = s * 8 + 2 * T + mm;
                if (m < nmem) {
                    float *zp = zb + (size_t)mem[m] * N + (warp + 8 * n) * 16 + G;
                    __stcg(zp, acc[n][s][mm]);
                    __stcg(zp + 8, acc[n][s][2 + mm]);
                }
            }
    return ok;
}

// Grouping of a window of at most 32 routing entries by one warp with votes (no block barrier, no shared atomics).
__device__ __forceinline__ void win_group_small(const WinArgs &a, WinShared &sh, int np) {
    const int lane = threadIdx.x & 31;
    const int e = lane < np ? __ldcg(a.picks + lane) : -1;
    const int row = lane / a.slots, slot = lane - row * a.slots;
    bool valid = lane < np && !expert_skipped(e, a.E, a.shared_exl3, a.e_lo, a.e_hi);
    for (int s = 0; s < a.slots - 1; ++s) {                   // a pick that repeats an earlier slot of its row names nothing
        const int o = __shfl_sync(0xffffffffu, e, min(row * a.slots + s, 31));
        if (s < slot && o == e) valid = false;
    }
    const uint32_t vmask = __ballot_sync(0xffffffffu, valid);
    const uint32_t same = __match_any_sync(0xffffffffu, valid ? e : -1 - lane) & vmask;   // valid lanes naming my expert
    const bool first = valid && (__ffs(same) - 1) == lane;
    const uint32_t fmask = __ballot_sync(0xffffffffu, first);
    int u = 0;                                                 // number of distinct experts with a smaller id
    for (int l = 0; l < 32; ++l) {
        const int o = __shfl_sync(0xffffffffu, e, l);
        if (((fmask >> l) & 1u) && o < e) ++u;
    }
    if (lane < np) sh.picks[lane] = e;
    if (valid) {
        sh.mem[u][__popc(same & ((1u << lane) - 1u))] = (unsigned short)lane;
        if (first) { sh.ids[u] = e; sh.cnt[u] = __popc(same); }
    }
    if (lane < a.rows) sh.rowlive[lane] = (vmask >> (lane * a.slots)) & (a.slots >= 32 ? 0xffffffffu : (1u << a.slots) - 1u);
    if (lane == 0) sh.U = __popc(fmask);
}

// =================================== service warp ===================================
template <int SETS>
__device__ __noinline__ void win_service_main(const WinArgs &a, WinShared &sh, unsigned char *smem, unsigned epoch, unsigned xepoch) {
    const int team = win_team(), lane = threadIdx.x & 31;
    unsigned char *tbase = smem + (size_t)team * WIN_TEAM_BYTES;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + (size_t)WIN_TEAMS * WIN_TEAM_BYTES) + team * WIN_BARS;
    uint64_t *done = full + WIN_NBUF * WIN_NG;
        // This team's contiguous share of each kind's items (teams numbered SM-major; the F items are dealt from the far
        // end so that they land on the teams with the fewest G and D items).
        const WinShape shp = win_shape(a.H, a.I, sh.U, a.rows);
        WinShared::Plan pl;
        {
            const unsigned nteams = gridDim.x * WIN_TEAMS, tg = blockIdx.x + gridDim.x * team, tr = nteams - 1 - tg;
            pl.g0 = (int)((unsigned)shp.n_g * tg / nteams);
            pl.d0 = (int)((unsigned)shp.n_d * tg / nteams);
            pl.f0 = (int)((unsigned)shp.n_f * tr / nteams);
            pl.ngl = (int)((unsigned)shp.n_g * (tg + 1) / nteams) - pl.g0;
            pl.nw = pl.ngl + (int)((unsigned)shp.n_d * (tg + 1) / nteams) - pl.d0;
            pl.nloc = pl.nw + (int)((unsigned)shp.n_f * (tr + 1) / nteams) - pl.f0;
        }
        // Requests the copies (lanes 0..7: one 2-KB row each) and publishes finished items: when the eight compute warps
        // are through with item q (their partial stores are issued, its buffer is free) the buffer is refilled with item
        // q + NBUF and the item's flag word takes the launch's epoch with a release store.
        auto issue = [&](int q, WinItem it) {
            const int b = q % WIN_NBUF, e = sh.ids[it.u()];
            const uint32_t *Tm = it.kind() ? a.dt : (it.mat() ? a.ut : a.gt);
            const int KT = (it.kind() ? a.I : a.H) >> 4, NT = (it.kind() ? a.H : a.I) >> 4;
            if (lane == 0)
                for (int g = 0; g < WIN_NG; ++g) mbar_expect_tx(full + b * WIN_NG + g, 4 * WIN_COLS * 8);
            if (lane < WIN_KTI) {
                const uint32_t *src = Tm + (((size_t)e * KT + it.split() * WIN_KTI + lane) * NT + (size_t)it.nb2() * 16) * 32;
                tma_load_1d(tbase + (size_t)b * WIN_WBUF + (size_t)lane * WIN_WROW, src, WIN_COLS * 8, full + b * WIN_NG + (lane >> 2));
            }
        };
        if (lane == 0) {
            sh.plan[team] = pl;
            if (team == 0) { sh.epoch = epoch; sh.xepoch = xepoch; }
        }
        __syncthreads();                          // the plans are there: the compute warps start staging
        int issued = 0;
        WinItem it_issue = win_pack(0, 0, 0, 0, 0);
        for (; issued < WIN_NBUF && issued < pl.nw; ++issued) {
            it_issue = win_local_next(shp, pl, issued, it_issue);
            issue(issued, it_issue);
        }
        WIN_STAMP_S(3);
        int q = 0;
        WinItem it_pub = win_pack(0, 0, 0, 0, 0);
        for (; q < pl.nw; ++q) {
            const int b = q % WIN_NBUF;
            it_pub = win_local_next(shp, pl, q, it_pub);
            bool ok = false;
            for (uint32_t i = 0; i < WIN_POLLS; ++i) {
                if (mbar_try_wait_hint(done + b, (uint32_t)(q / WIN_NBUF) & 1u, 1000u)) { ok = true; break; }
                if ((i & 63u) == 63u && *reinterpret_cast<volatile int *>(&sh.abort[team])) break;
            }
            if (!ok) break;
            WIN_STAMP_S(32 + q * 3);
            if (issued < pl.nw) {
                it_issue = win_local_next(shp, pl, issued, it_issue);
                issue(issued, it_issue);
                ++issued;
            }
            WIN_STAMP_S(33 + q * 3);
            if (lane == 0) {
                const int e = sh.ids[it_pub.u()];
                st_release_gpu(it_pub.kind() ? win_fd(a, e, it_pub.nb2()) + it_pub.split()
                                             : win_fg(a, e, it_pub.nb2()) + it_pub.mat() * shp.SKg + it_pub.split(), epoch);
            }
            __syncwarp();
            WIN_STAMP_S(34 + q * 3);
        }
        if (q < pl.nw) {
            // a give-up somewhere in the team: leave no copy in flight (the buffers are this CTA's shared memory)
            if (lane == 0 && !*reinterpret_cast<volatile int *>(&sh.abort[team])) { atomicExch(a.status, GF_STATUS_TMA_TIMEOUT); sh.abort[team] = 1; }
            for (int k = q; k < issued; ++k)
                for (int g = 0; g < WIN_NG; ++g) win_mbar_drain(full + (k % WIN_NBUF) * WIN_NG + g, (uint32_t)(k / WIN_NBUF) & 1u);
        }
}

// =================================== compute warps ===================================
template <int SETS>
__device__ __noinline__ void win_compute_main(const WinArgs &a, WinShared &sh, unsigned char *smem) {
    __syncthreads();                              // the plans are there
    // Only q, the packed item and the key of the current run stay in registers from item to item; everything else is
    // derived again per item from the thread index, the kernel arguments and the plan in shared memory.
    uint32_t cur_key = 0xffffffffu;
    WinItem it = win_pack(0, 0, 0, 0, 0);
#pragma unroll 1
    for (int q = 0;; ++q) {
        const int team_ = win_opaque((int)(threadIdx.x >> 5)) / WIN_TEAM_WARPS;
        {
            const volatile WinShared::Plan &vp = sh.plan[team_];
            WinShared::Plan pl;
            pl.g0 = vp.g0; pl.d0 = vp.d0; pl.f0 = vp.f0; pl.ngl = vp.ngl; pl.nw = vp.nw; pl.nloc = vp.nloc;
            if (q >= pl.nloc) break;
            const WinShape shp = win_shape(win_opaque(a.H), win_opaque(a.I), *reinterpret_cast<volatile int *>(&sh.U), a.rows);
            it = win_local_next(shp, pl, q, it);
            unsigned char *tb = smem + (size_t)team_ * WIN_TEAM_BYTES;
            uint32_t *act_ = reinterpret_cast<uint32_t *>(tb + WIN_NBUF * WIN_WBUF);
            float *scr_ = reinterpret_cast<float *>(tb + WIN_NBUF * WIN_WBUF + WIN_ACT);
            WIN_STAMP(4 + q * 4);
            if (it.kind() == 2) {
                // ---- F item: the pairs of (row, 128-column block) are finished and combined
                if (q == pl.nw) team_bar(team_);               // the last K loop of the team has read the staged operands
#ifndef WIN_EXP_NOEPI
                if (!win_finish_block(a, sh, reinterpret_cast<float *>(act_), scr_, it.u(), it.nb2(), team_,
                                      *reinterpret_cast<volatile unsigned *>(&sh.epoch), *reinterpret_cast<volatile unsigned *>(&sh.xepoch)))
                    break;
#else
                if (win_warp() == 0)
                    win_block_out(a, sh, team_, it.u(), it.nb2(), make_float4(0.f, 0.f, 0.f, 0.f), *reinterpret_cast<volatile unsigned *>(&sh.epoch),
                                  *reinterpret_cast<volatile unsigned *>(&sh.xepoch));
#endif
                WIN_STAMP(5 + q * 4);
                continue;
            }
            if (it.run_key() != cur_key) {
                // ---- a new run: stage the members' activations of this K range once for all its items
                cur_key = it.run_key();
                const int e = sh.ids[it.u()], nmem = sh.cnt[it.u()];
                const unsigned short *mem = sh.mem[it.u()];
                team_bar(team_);                               // every warp is through with the K loops of the run before
                if (it.kind() == 0) {
                    win_stage_rotate<SETS>(a, act_, mem, nmem, e, it.mat(), it.split() * WIN_KC);
                } else {
                    // the 2 x H/128 gate and up partials of these 128 columns of the intermediate must be there
                    if (win_warp() == 0 && !win_wait_flags(win_fg(a, e, it.split() >> 1), 2 * shp.SKg, *reinterpret_cast<volatile unsigned *>(&sh.epoch))) {
                        if ((threadIdx.x & 31) == 0) { atomicExch(a.status, GF_STATUS_PEER_TIMEOUT); sh.abort[team_] = 1; }
                    }
                    team_bar(team_);
                    if (sh.abort[team_]) break;
                    WIN_STAMP(5 + q * 4);
#ifndef WIN_EXP_NOEPI
                    win_stage_swiglu<SETS>(a, sh, act_, scr_, mem, nmem, e, it.split(), team_);
#endif
                }
                team_bar(team_);
                WIN_STAMP(6 + q * 4);
            }
        }

        // ---- the K loop, and this split's partial of every member to its fixed place in global scratch (its operands
        //      are derived here, after the staging, so that they do not occupy registers during it)
        {
            const int team2 = win_opaque((int)(threadIdx.x >> 5)) / WIN_TEAM_WARPS;
            const int H2 = win_opaque(a.H), I2 = win_opaque(a.I);
            unsigned char *tb = smem + (size_t)team2 * WIN_TEAM_BYTES;
            uint64_t *full2 = reinterpret_cast<uint64_t *>(smem + (size_t)WIN_TEAMS * WIN_TEAM_BYTES) + team2 * WIN_BARS;
            const int kind = it.kind(), u = it.u();
            const int N = kind ? H2 : I2, b = q % WIN_NBUF;
            float *Z = kind ? a.z2 : a.z1;
            const int zs = kind ? it.split() : it.mat() * (H2 / WIN_KC) + it.split();
            const bool ok = win_kloop<SETS>(tb + (size_t)b * WIN_WBUF, reinterpret_cast<const uint32_t *>(tb + WIN_NBUF * WIN_WBUF), full2 + b * WIN_NG,
                                            (uint32_t)(q / WIN_NBUF) & 1u, sh.cnt[u], sh.mem[u],
                                            Z + (size_t)zs * (a.rows * a.slots) * N + it.nb2() * WIN_COLS, N);
            __syncwarp();
            if ((threadIdx.x & 31) == 0) {
                const int team3 = win_team();
                if (!ok) { atomicExch(a.status, GF_STATUS_TMA_TIMEOUT); sh.abort[team3] = 1; }
                // this warp's partial stores are issued; it has left the buffer
                mbar_arrive(reinterpret_cast<uint64_t *>(smem + (size_t)WIN_TEAMS * WIN_TEAM_BYTES) + team3 * WIN_BARS + WIN_NBUF * WIN_NG + q % WIN_NBUF);
            }
            WIN_STAMP(7 + q * 4);
            if (!ok) break;
        }
    }
    WIN_STAMP(31);
    if (a.peers.world > 1) {
        team_bar(win_team());
        win_exchange_sum(a, sh, win_team(), sh.epoch, sh.xepoch);
    }
}

template <int SETS>
__global__ void __launch_bounds__(WIN_THREADS, 1) window_kernel(const __grid_constant__ WinArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ WinShared sh;

    const int tid = threadIdx.x, team = win_team(), warp = win_warp(), lane = tid & 31;
    const bool service = warp == WIN_CW;
    unsigned char *tbase = smem + (size_t)team * WIN_TEAM_BYTES;
    // per team: full[buffer][group] count copied bytes; done[buffer] counts the compute warps that are through with it
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + (size_t)WIN_TEAMS * WIN_TEAM_BYTES) + team * WIN_BARS;
    uint64_t *done = full + WIN_NBUF * WIN_NG;

    WIN_STAMP(0);
    if (service && lane == 0) {
        for (int k = 0; k < WIN_NBUF * WIN_NG; ++k) mbar_init(full + k, 1);
        for (int k = 0; k < WIN_NBUF; ++k) mbar_init(done + k, WIN_CW);
        mbar_fence_init();
        sh.abort[team] = 0; sh.qn[team] = 0;
    }
    const int np = a.rows * a.slots;
    pdl_launch_dependents();
    pdl_wait();                                   // the routing table and the layer input may belong to the kernel before
    WIN_STAMP(1);
    const unsigned epoch = __ldcg(a.sync) + 1u;
    // the exchange counts on its own: every rank advances it once per exchange, whichever owners computed the layers
    const unsigned xepoch = a.peers.world > 1 ? __ldcg(a.peers.epoch) + 1u : 0u;

    // ---- grouping (native/grouping.cu:67-100 semantics): distinct experts computed here in ascending id order, their
    //      members in ascending row order.  A pick that repeats an earlier slot of its row names nothing.
    if (np <= 32) {
        if (tid < 32) win_group_small(a, sh, np);
        __syncthreads();
    } else {
        if (tid < 32) sh.used[tid] = 0u;
        if (tid < 16) sh.rowlive[tid] = 0u;
        if (tid < WIN_UMAX) sh.cnt[tid] = 0;
        if (tid < np) sh.picks[tid] = __ldcg(a.picks + tid);
        __syncthreads();
        int my_e = -1, my_row = 0;
        bool valid = false;
        if (tid < np) {
            my_row = tid / a.slots;
            const int my_slot = tid - my_row * a.slots;
            my_e = sh.picks[tid];
            valid = !expert_skipped(my_e, a.E, a.shared_exl3, a.e_lo, a.e_hi);
            for (int s = 0; s < my_slot; ++s) valid = valid && sh.picks[my_row * a.slots + s] != my_e;
            if (valid) {
                atomicOr(&sh.used[my_e >> 5], 1u << (my_e & 31));
                atomicOr(&sh.rowlive[my_row], 1u << my_slot);
            }
        }
        __syncthreads();
        if (tid < 32) {
            const int c = __popc(sh.used[tid]);
            int incl = c;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += up;
            }
            sh.base[tid] = incl - c;
            if (tid == 31) sh.U = min(incl, WIN_UMAX);
        }
        __syncthreads();
        if (valid) {
            const int u = sh.base[my_e >> 5] + __popc(sh.used[my_e >> 5] & ((1u << (my_e & 31)) - 1u));
            int pos = 0;
            for (int r = 0; r < my_row; ++r) {
                bool has = false;
                for (int s = 0; s < a.slots; ++s) has = has || sh.picks[r * a.slots + s] == my_e;
                pos += has;
            }
            if (u < WIN_UMAX) {
                sh.mem[u][pos] = (unsigned short)tid;
                if (pos == 0) sh.ids[u] = my_e;
                atomicAdd(&sh.cnt[u], 1);
            }
        }
        __syncthreads();
    }
    WIN_STAMP(2);

    if (service) win_service_main<SETS>(a, sh, smem, epoch, xepoch);
    else win_compute_main<SETS>(a, sh, smem);
}

bool experts_window_supported(const glmflash_config &c, int rows) {
    const int umax = std::min(rows * (c.slots - 1) + 1, c.experts + 1);
    // (an owner of the shared expert that is decided per window, shared_exl3 == 2, is served by the three-launch kernels)
    return rows >= 1 && rows <= 16 && rows * c.slots <= 512 && umax <= WIN_UMAX && c.hidden <= 8192 && c.inter <= 8192 &&
           c.shared_exl3 != 2;
}

size_t experts_window_sync_words(const glmflash_config &c) { return win_sync_words(c.experts, c.hidden, c.inter); }

int experts_run_window(glmflash_experts *e, cudaStream_t s, const glmflash_weights *w, const void *input, int x_stride,
                       const int32_t *picks, const float *route_w, int rows, float *out, const WinPeers *peers,
                       int shared_here) {
    const glmflash_config &c = e->cfg;
    GF_REQUIRE(rows > 0 && rows <= c.max_rows, "expert verifier row/member bounds");
    GF_REQUIRE(experts_window_supported(c, rows), "window shape outside the one-launch layer kernel's tables");
    GF_REQUIRE(x_stride >= c.hidden && x_stride % 4 == 0, "x_stride must be >= hidden and a multiple of 4");
    GF_REQUIRE(((uintptr_t)w->gt | (uintptr_t)w->ut | (uintptr_t)w->dt) % 16 == 0, "trellis tensors must be 16-byte aligned");
    GF_REQUIRE(((uintptr_t)input | (uintptr_t)w->suh_g | (uintptr_t)w->suh_u | (uintptr_t)w->suh_d | (uintptr_t)w->svh_g |
                (uintptr_t)w->svh_u | (uintptr_t)w->svh_d) % 8 == 0, "input and scale vectors must be 8-byte aligned");
    GF_REQUIRE(e->z1 && e->z2 && e->sync && out, "owner has no window scratch");
    WinArgs a{};
    a.x = (const __nv_bfloat16 *)input; a.picks = picks; a.route_w = route_w;
    a.gt = w->gt; a.ut = w->ut; a.dt = w->dt;
    a.suh_g = (const __half *)w->suh_g; a.suh_u = (const __half *)w->suh_u; a.suh_d = (const __half *)w->suh_d;
    a.svh_g = (const __half *)w->svh_g; a.svh_u = (const __half *)w->svh_u; a.svh_d = (const __half *)w->svh_d;
    a.xd = e->xd; a.z1 = e->z1; a.z2 = e->z2; a.y = e->y; a.out = out;
    a.sync = e->sync; a.status = e->status;
    a.rows = rows; a.slots = c.slots; a.H = c.hidden; a.I = c.inter; a.E = c.experts; a.e_lo = c.expert_lo; a.e_hi = c.expert_hi;
    a.shared_exl3 = shared_here < 0 ? c.shared_exl3 : (shared_here != 0);
    a.x_stride = x_stride; a.limit = c.limit;
    if (peers) a.peers = *peers;
    else { a.peers = WinPeers{}; a.peers.world = 1; }
    int dev = 0;
    GF_CUDA(cudaGetDevice(&dev));
    static bool configured[64][2] = {};
    const int sets = rows > 8 ? 2 : 1;
    if (!configured[dev & 63][sets - 1]) {
        if (sets == 1) GF_CUDA(cudaFuncSetAttribute(window_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WIN_SMEM));
        else GF_CUDA(cudaFuncSetAttribute(window_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WIN_SMEM));
        configured[dev & 63][sets - 1] = true;
    }
    if (!e->sm_count) GF_CUDA(cudaDeviceGetAttribute(&e->sm_count, cudaDevAttrMultiProcessorCount, dev));
    const dim3 grid((unsigned)e->sm_count), block(WIN_THREADS);
    if (sets == 1) return launch_k(window_kernel<1>, grid, block, WIN_SMEM, s, c.pdl != 0, a);
    return launch_k(window_kernel<2>, grid, block, WIN_SMEM, s, c.pdl != 0, a);
}

}  // namespace gf

#ifdef WIN_TRACE
extern "C" int glmflash_win_trace_set(long long *buffer) {
    GF_CUDA(cudaMemcpyToSymbol(gf::g_win_trace, &buffer, sizeof(buffer)));
    return 0;
}
#endif
