// Expert-parallel combine fused with its exchange over NVLink (one process per GPU).
//
// Upstream gathers every rank's fp32 partial layer output with an all-gather (NCCL, or its one-shot RoCE gather
// kernel, native/roce.cu:217-371) and then adds the ranks' rows in fixed rank order (src/model.rs:485-496,
// src/comm.rs:1-2).  Here one kernel per rank does the whole step:
//   1. combine: partial[r][:] = sum of this rank's pairs of row r (weights applied), as combine_kernel;
//   2. push:    the partial is stored straight into slot `rank` of EVERY peer's receive buffer through peer-mapped
//               pointers (plain st.global over NVLink, no multicast), then a release fence and one flag word per
//               (source rank, CTA) carries the epoch;
//   3. wait:    the same CTA spins (bounded) on its own GPU's flags until every source has delivered the epoch;
//   4. sum:     the slots are added in ascending rank order -- the reference's determinism rule -- into out.
// Windows of <= 16 rows send flag and data in ONE 8-byte word (ep_combine_ll_kernel: every fp32 travels as the pair
// {value, epoch}, an aligned 8-byte store arrives whole, and the receiver polls the words themselves), which takes the
// fence and the separate flag round trip out of the latency: the push costs one NVLink crossing.
// Windows of more than 16 rows use a two-step form of the same kernel (ep_exchange_rows_kernel): every row has
// one owner rank (chunks of 8 rows, dealt out in contiguous runs); every rank stores its partial of the row only into the
// OWNER's receive slot, the owner
// adds the slots in rank order and stores the finished row into every rank's result buffer, and every rank waits for
// that.  Per rank about 2 x rows x H x 4 bytes cross NVLink instead of world x that (268 MB at 4096 rows on 8 GPUs);
// with glmflash_ep_set_exchange_bf16 the first of the two steps moves bf16 (1.5 x rows x H x 4 bytes in all).
// (the owner stores them straight into the peers' output rows, which live inside the mapped area).
// Receive buffers are double-buffered by epoch parity; the epoch lives in device memory and is advanced by the
// last CTA of a call, so captured graphs replay correctly.  A wait that gives up sets the status word (the
// analogue of upstream's poison word, native/roce.cu:127-141) and the kernel returns; nothing spins unbounded.
#include <new>
#include <vector>

#include "common.cuh"
#include "owners.cuh"

namespace gf {

constexpr int EP_MAX_WORLD = 8;
constexpr int EP_THREADS = 256;

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct EpPeers {
    float *recv[EP_MAX_WORLD];          // recv[k]: rank k's receive buffer [2][world][max_rows][H] (peer-mapped)
    unsigned *flags[EP_MAX_WORLD];      // flags[k]: rank k's flags [2][world][max_ctas]
    float *fin[EP_MAX_WORLD];           // fin[k]: rank k's output rows [max_rows][H]               (two-step form)
    unsigned *fin_flags[EP_MAX_WORLD];  // fin_flags[k]: rank k's [2][max_ctas]                     (two-step form)
    uint2 *ll[EP_MAX_WORLD];            // ll[k]: rank k's {value, epoch} words [2][world][max_rows][H]  (<= 16 rows)
};

// This rank's partial of row r, columns d..d+3: its computed pairs of the row, weights applied, ascending slots.
__device__ __forceinline__ float4 ep_partial(const float *__restrict__ Y, const int *__restrict__ picks,
                                             const float *__restrict__ route_w, int r, int d, int slots, int H, int E,
                                             int shared_exl3, int e_lo, int e_hi, int srow_lo, int srow_hi) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < slots; ++s) {
        const int e = picks[r * slots + s];
        bool skip = e < 0 || e > E || (e == E ? !shared_exl3 : (e < e_lo || e >= e_hi));
        if (e == E && srow_hi > srow_lo && (r < srow_lo || r >= srow_hi)) skip = true;      // shared expert: row window
        if (skip) continue;
        const float4 y = *reinterpret_cast<const float4 *>(Y + ((size_t)r * slots + s) * H + d);
        if (s == slots - 1) { acc.x += y.x; acc.y += y.y; acc.z += y.z; acc.w += y.w; }
        else {
            const float w = route_w[r * slots + s];
            acc.x += w * y.x; acc.y += w * y.y; acc.z += w * y.z; acc.w += w * y.w;
        }
    }
    return acc;
}

// Bounded wait for *f == epoch.  Gives up at once when another wait of this call has already run out.
__device__ __forceinline__ bool ep_wait(const unsigned *f, unsigned epoch, unsigned wait_polls, int *status) {
    for (unsigned i = 0; i < wait_polls; ++i) {
        if (ld_acquire_sys(f) == epoch) return true;
        if ((i & 1023u) == 1023u) {
            if (*reinterpret_cast<volatile int *>(status) == GF_STATUS_PEER_TIMEOUT) break;
            __nanosleep(200);
        }
    }
    atomicExch(status, GF_STATUS_PEER_TIMEOUT);
    return false;
}

__global__ void __launch_bounds__(EP_THREADS) ep_combine_kernel(const float *__restrict__ Y, const int *__restrict__ picks,
                                                                const float *__restrict__ route_w, float *__restrict__ out,
                                                                EpPeers peers, unsigned *epoch_ptr, unsigned *done_ptr,
                                                                int *status, int rank, int world, int rows, int max_rows,
                                                                int max_ctas, int slots, int H, int E, int shared_exl3,
                                                                int e_lo, int e_hi, int srow_lo, int srow_hi,
                                                                unsigned wait_polls) {
    // (the routing table was complete before the expert kernels in front ran: it may be read ahead of the dependency wait)
    __shared__ uint32_t used_sh[32];
    if (shared_exl3 == 2) shared_exl3 = shared_owner_of_window(picks, rows * slots, E, e_hi - e_lo, used_sh) == e_lo / (e_hi - e_lo);
    pdl_wait();
    pdl_launch_dependents();
    __shared__ int ok_sh;
    const int r = blockIdx.y;
    const int cta = blockIdx.y * gridDim.x + blockIdx.x;
    const int d = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const unsigned epoch = *epoch_ptr + 1u;                   // every CTA reads it before the last one advances it
    const unsigned par = epoch & 1u;
    const size_t slot_elems = (size_t)max_rows * H;
    if (d < H) {
        // 1. this rank's partial of row r; 2. push into slot `rank` of every rank's receive buffer (its own included)
        const float4 acc = ep_partial(Y, picks, route_w, r, d, slots, H, E, shared_exl3, e_lo, e_hi, srow_lo, srow_hi);
        for (int k = 0; k < world; ++k) {
            float *dst = peers.recv[k] + ((size_t)par * world + rank) * slot_elems + (size_t)r * H + d;
            *reinterpret_cast<float4 *>(dst) = acc;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < world)
        st_release_sys(peers.flags[threadIdx.x] + ((size_t)par * world + rank) * max_ctas + cta, epoch);
    // 3. wait for every source's copy of this CTA's region
    if (threadIdx.x == 0) ok_sh = 1;
    __syncthreads();
    if (threadIdx.x < world)
        if (!ep_wait(peers.flags[rank] + ((size_t)par * world + threadIdx.x) * max_ctas + cta, epoch, wait_polls, status)) ok_sh = 0;
    __syncthreads();
    // 4. ordered sum
    if (d < H && ok_sh) {
        const float *src = peers.recv[rank] + (size_t)par * world * slot_elems + (size_t)r * H + d;
        float4 sum = __ldcg(reinterpret_cast<const float4 *>(src));
        for (int k = 1; k < world; ++k) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(src + (size_t)k * slot_elems));
            sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        }
        *reinterpret_cast<float4 *>(out + (size_t)r * H + d) = sum;
    }
    // the last CTA of the call advances the epoch (after every CTA has read it)
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned n = gridDim.x * gridDim.y;
        if (atomicAdd(done_ptr, 1u) == n - 1u) {
            *done_ptr = 0u;
            __threadfence();
            *epoch_ptr = epoch;
        }
    }
}

// Windows of <= 16 rows, flag-in-data form.  A thread owns four columns of a row: it stores its partial as four
// {value, epoch} words into slot `rank` of every PEER (two 16-byte volatile stores each; an aligned 8-byte word is
// never torn), then adds the slots in ascending rank order, taking its own partial from registers and polling the
// peers' words in its own GPU's memory until both halves of each 16-byte load carry the epoch.  Epochs start at 1 and
// the buffers start zeroed; a slot is rewritten two epochs later, after its reader has finished (the writer cannot
// finish the epoch in between without the reader's data of that epoch).
__device__ __forceinline__ void st_volatile_v4(uint2 *p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const uint2 *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__global__ void __launch_bounds__(EP_THREADS) ep_combine_ll_kernel(const float *__restrict__ Y, const int *__restrict__ picks,
                                                                   const float *__restrict__ route_w, float *__restrict__ out,
                                                                   EpPeers peers, unsigned *epoch_ptr, unsigned *done_ptr,
                                                                   int *status, int rank, int world, int rows, int max_rows,
                                                                   int slots, int H, int E, int shared_exl3, int e_lo, int e_hi,
                                                                   unsigned wait_polls) {
    // (the routing table was complete before the expert kernels in front ran: it may be read ahead of the dependency wait)
    __shared__ uint32_t used_sh[32];
    if (shared_exl3 == 2) shared_exl3 = shared_owner_of_window(picks, rows * slots, E, e_hi - e_lo, used_sh) == e_lo / (e_hi - e_lo);
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.y;
    const int d = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const unsigned epoch = *epoch_ptr + 1u;                   // every CTA reads it before the last one advances it
    const unsigned par = epoch & 1u;
    const size_t slot_words = (size_t)max_rows * H;
    if (d < H) {
        const float4 acc = ep_partial(Y, picks, route_w, r, d, slots, H, E, shared_exl3, e_lo, e_hi, 0, 0);
        const size_t at = (size_t)r * H + d;
        for (int k = 0; k < world; ++k) {
            if (k == rank) continue;
            uint2 *dst = peers.ll[k] + ((size_t)par * world + rank) * slot_words + at;
            st_volatile_v4(dst, __float_as_uint(acc.x), epoch, __float_as_uint(acc.y), epoch);
            st_volatile_v4(dst + 2, __float_as_uint(acc.z), epoch, __float_as_uint(acc.w), epoch);
        }
        // all peers' words are requested together and only the late ones are asked for again: the wait costs one local
        // round trip after the last arrival, not one per peer
        uint4 lo[EP_MAX_WORLD], hi[EP_MAX_WORLD];
        unsigned missing = ((1u << world) - 1u) & ~(1u << rank);
        bool ok = true;
        for (unsigned i = 0; missing; ++i) {
            if (i >= wait_polls) { ok = false; break; }
            if ((i & 1023u) == 1023u) {
                if (*reinterpret_cast<volatile int *>(status) == GF_STATUS_PEER_TIMEOUT) { ok = false; break; }
                __nanosleep(200);
            }
#pragma unroll
            for (int k = 0; k < EP_MAX_WORLD; ++k)
                if (missing >> k & 1u) {
                    const uint2 *src = peers.ll[rank] + ((size_t)par * world + k) * slot_words + at;
                    lo[k] = ld_volatile_v4(src);
                    hi[k] = ld_volatile_v4(src + 2);
                }
#pragma unroll
            for (int k = 0; k < EP_MAX_WORLD; ++k)
                if ((missing >> k & 1u) && lo[k].y == epoch && lo[k].w == epoch && hi[k].y == epoch && hi[k].w == epoch)
                    missing &= ~(1u << k);
        }
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < EP_MAX_WORLD; ++k) {
            if (k >= world) break;
            const float4 v = k == rank ? acc
                                       : make_float4(__uint_as_float(lo[k].x), __uint_as_float(lo[k].z), __uint_as_float(hi[k].x),
                                                     __uint_as_float(hi[k].z));
            if (k == 0) sum = v;
            else { sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w; }
        }
        if (ok) *reinterpret_cast<float4 *>(out + at) = sum;
        else atomicExch(status, GF_STATUS_PEER_TIMEOUT);
    }
    // the last CTA of the call advances the epoch (after every CTA has read it)
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned n = gridDim.x * gridDim.y;
        if (atomicAdd(done_ptr, 1u) == n - 1u) {
            *done_ptr = 0u;
            __threadfence();
            *epoch_ptr = epoch;
        }
    }
}

// Two-step form for large windows (see the head of this file).  CTA = chunk of EP_RB consecutive rows, all columns; a
// chunk has one owner rank (the owners' row ranges are multiples of EP_RB), so one fence and one flag per chunk and step
// replace one per row.  A CTA only ever waits for the CTAs of the SAME chunk on other ranks, and every rank walks the
// chunks in the same order, so no wait depends on a CTA that is dispatched later on its own GPU.
// BF16: the partials of step 1 cross NVLink as bf16 (upstream casts every rank's rows to bf16 before its gather and adds
// them in fp32, src/batch.rs:651-658); every rank's partial, the owner's own included, takes the same rounding, so the
// sum still depends on nothing but the rank order.  The finished rows of step 2 stay fp32.
constexpr int EP_RB_MAX = 32;
__device__ __forceinline__ uint2 ep_pack_bf16(const float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    return make_uint2(*reinterpret_cast<const uint32_t *>(&a), *reinterpret_cast<const uint32_t *>(&b));
}
__device__ __forceinline__ float4 ep_unpack_bf16(const uint2 w) {
    return make_float4(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xffff0000u), __uint_as_float(w.y << 16),
                       __uint_as_float(w.y & 0xffff0000u));
}
template <bool BF16>
__global__ void __launch_bounds__(EP_THREADS, 4) ep_exchange_rows_kernel(const float *__restrict__ Y, const int *__restrict__ picks,
                                                                      const float *__restrict__ route_w, float *__restrict__ out,
                                                                      EpPeers peers, unsigned *epoch_ptr, unsigned *done_ptr,
                                                                      int *status, int rank, int world, int rows, int max_rows,
                                                                      int max_ctas, int slots, int H, int E, int shared_exl3,
                                                                      int e_lo, int e_hi, int srow_lo, int srow_hi,
                                                                      unsigned wait_polls, int EP_RB) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ int ok_sh;
    const int chunk = blockIdx.x, r0 = chunk * EP_RB, r1 = min(r0 + EP_RB, rows);
    const unsigned epoch = *epoch_ptr + 1u;
    const unsigned par = epoch & 1u;
    const size_t slot_elems = (size_t)max_rows * H;
    const int chunks = (rows + EP_RB - 1) / EP_RB, per = (chunks + world - 1) / world;
    const int owner = chunk / per;                            // < world because chunk < chunks
    const int q4 = H >> 2, items = (r1 - r0) * q4;            // float4 pieces of the chunk
    // 1. this rank's partial of the chunk goes to the owner's slot `rank`.  Which pairs of a row are this rank's is looked
    //    up once per (row, slot) into shared memory; a thread then has the loads of all its pairs of a piece in flight
    //    together (the decision is uniform over a warp: a warp works on one row), and adds them in ep_partial's order.
    __shared__ unsigned char take_sh[EP_RB_MAX][32];               // 1: pair (row, slot) is this rank's
    for (int i = threadIdx.x; i < (r1 - r0) * slots; i += EP_THREADS) {
        const int r = r0 + i / slots, sl = i % slots;
        const int e = picks[r * slots + sl];
        bool skip = e < 0 || e > E || (e == E ? !shared_exl3 : (e < e_lo || e >= e_hi));
        if (e == E && srow_hi > srow_lo && (r < srow_lo || r >= srow_hi)) skip = true;
        take_sh[i / slots][sl] = skip ? 0 : 1;
    }
    __syncthreads();
    {
        float *slot = peers.recv[owner] + ((size_t)par * world + rank) * slot_elems;
#pragma unroll 2
        for (int i = threadIdx.x; i < items; i += EP_THREADS) {
            const int rl = i / q4, r = r0 + rl, d = (i % q4) * 4;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s0 = 0; s0 < slots; s0 += 8) {
                float4 y[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (s0 + j < slots && take_sh[rl][s0 + j])
                        y[j] = __ldcs(reinterpret_cast<const float4 *>(Y + ((size_t)r * slots + s0 + j) * H + d));
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (s0 + j >= slots || !take_sh[rl][s0 + j]) continue;
                    if (s0 + j == slots - 1) { acc.x += y[j].x; acc.y += y[j].y; acc.z += y[j].z; acc.w += y[j].w; }
                    else {
                        const float w = route_w[r * slots + s0 + j];
                        acc.x += w * y[j].x; acc.y += w * y[j].y; acc.z += w * y[j].z; acc.w += w * y[j].w;
                    }
                }
            }
            if (BF16) *reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(slot) + (size_t)r * H + d) = ep_pack_bf16(acc);
            else *reinterpret_cast<float4 *>(slot + (size_t)r * H + d) = acc;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) { st_release_sys(peers.flags[owner] + ((size_t)par * world + rank) * max_ctas + chunk, epoch); ok_sh = 1; }
    __syncthreads();
    // 2. the owner adds the slots in rank order and stores the finished rows into every rank's result buffer
    if (owner == rank) {
        if (threadIdx.x < world)
            if (!ep_wait(peers.flags[rank] + ((size_t)par * world + threadIdx.x) * max_ctas + chunk, epoch, wait_polls, status)) ok_sh = 0;
        __syncthreads();
        if (ok_sh)
#pragma unroll 2
            for (int i = threadIdx.x; i < items; i += EP_THREADS) {
                const size_t off = (size_t)(r0 + i / q4) * H + (i % q4) * 4;
                const float *base = peers.recv[rank] + (size_t)par * world * slot_elems;
                auto slot_value = [&](int k) {
                    if (BF16)
                        return ep_unpack_bf16(__ldcg(reinterpret_cast<const uint2 *>(
                            reinterpret_cast<const __nv_bfloat16 *>(base + (size_t)k * slot_elems) + off)));
                    return __ldcg(reinterpret_cast<const float4 *>(base + (size_t)k * slot_elems + off));
                };
                float4 sum = slot_value(0);
                for (int k = 1; k < world; ++k) {
                    const float4 v = slot_value(k);
                    sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
                }
                for (int k = 0; k < world; ++k) *reinterpret_cast<float4 *>(peers.fin[k] + off) = sum;
            }
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x < world && ok_sh) st_release_sys(peers.fin_flags[threadIdx.x] + (size_t)par * max_ctas + chunk, epoch);
    }
    // 3. everyone waits for the finished chunk: its owner has stored it straight into this rank's output rows.  (The
    //    output needs no second buffer: an owner finishes a chunk of the NEXT call only after this rank's partial of that
    //    call, which this rank sends after everything it enqueued behind this call -- the readers of the output -- has run.)
    if (threadIdx.x == 0)
        if (!ep_wait(peers.fin_flags[rank] + (size_t)par * max_ctas + chunk, epoch, wait_polls, status)) ok_sh = 0;
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(done_ptr, 1u) == gridDim.x - 1u) {
            *done_ptr = 0u;
            __threadfence();
            *epoch_ptr = epoch;
        }
    }
}
}  // namespace gf

using namespace gf;

struct glmflash_ep {
    glmflash_config cfg;
    int rank = 0, world = 1, max_ctas = 0;
    unsigned char *local = nullptr;               // one allocation: recv | flags | epoch | done | status
    size_t recv_bytes = 0, flag_bytes = 0, fin_bytes = 0, fin_flag_bytes = 0, win_flag_bytes = 0, ll_bytes = 0, total_bytes = 0;
    size_t ll_offset() const { return recv_bytes + flag_bytes + fin_bytes + fin_flag_bytes + win_flag_bytes; }
    size_t tail() const { return ll_offset() + ll_bytes; }   // epoch | done | status
    void *peer_base[EP_MAX_WORLD] = {};
    bool opened[EP_MAX_WORLD] = {};
    bool connected = false;
    float *out = nullptr;
    unsigned wait_polls = 2000000u;               // about a second of polling before a wait gives up
    int chunk_rows = 8;                           // rows per chunk of the two-step form (every rank the same)
    bool use_ll = true;                           // windows of <= 16 rows: flag-in-data words (GLMFLASH_EP_LL=0: fence + flag)
    bool bf16_rows = false;                       // windows of more than 16 rows: partials cross NVLink as bf16
};

// What a rank publishes: the IPC handle of its receive area and a hash of everything the peers' address arithmetic
// depends on.  Upstream makes its ranks agree on their configuration with control records before the first exchange
// (src/comm.rs:66-96, src/model.rs:259-315); here the agreement rides on the bootstrap blob.
struct EpBlob {
    cudaIpcMemHandle_t mem;
    uint64_t config_hash;
};
static uint64_t ep_config_hash(const glmflash_config &c, int world, int chunk_rows, bool use_ll) {
    constexpr int32_t EP_LAYOUT = 4;                          // bumped whenever the mapped area's layout or protocol changes
    const int32_t f[8] = {GLMFLASH_ABI_VERSION * 256 + EP_LAYOUT, c.hidden, c.inter, c.experts, c.slots, c.max_rows, world, EP_THREADS | chunk_rows << 12 | (use_ll ? 1 << 20 : 0)};
    uint64_t h = 1469598103934665603ull;                      // FNV-1a
    for (size_t i = 0; i < sizeof(f); ++i) {
        h ^= reinterpret_cast<const unsigned char *>(f)[i];
        h *= 1099511628211ull;
    }
    return h;
}
extern "C" size_t glmflash_ep_handle_bytes(void) { return sizeof(EpBlob); }

extern "C" int glmflash_ep_new(const glmflash_config *cfg, size_t cfg_bytes, int rank, int world, glmflash_ep **out) {
    GF_REQUIRE(out != nullptr, "out is null");
    *out = nullptr;
    if (check_config(cfg, cfg_bytes, 8192)) return -1;
    GF_REQUIRE(world >= 1 && world <= EP_MAX_WORLD && rank >= 0 && rank < world, "rank / world out of range (world <= 8)");
    glmflash_ep *h = new (std::nothrow) glmflash_ep();
    GF_REQUIRE(h != nullptr, "out of host memory");
    h->cfg = *cfg; h->rank = rank; h->world = world;
    if (const char *v = getenv("GLMFLASH_EP_LL")) h->use_ll = atoi(v) != 0;      // comparison runs
    if (const char *v = getenv("GLMFLASH_EP_CHUNK_ROWS")) h->chunk_rows = std::min(std::max(atoi(v), 1), EP_RB_MAX);
    const size_t H = cfg->hidden, R = cfg->max_rows;
    h->max_ctas = (int)(((H / 4 + EP_THREADS - 1) / EP_THREADS) * R);
    h->recv_bytes = (size_t)2 * world * R * H * 4;
    h->flag_bytes = ((size_t)2 * world * h->max_ctas * 4 + 255) / 256 * 256;
    h->fin_bytes = R > 16 ? (size_t)R * H * 4 : 0;            // the two-step form (windows of more than 16 rows) keeps its
                                                              // output rows inside the mapped area: owners store into them
    h->fin_flag_bytes = R > 16 ? ((size_t)2 * h->max_ctas * 4 + 255) / 256 * 256 : 0;
    // arrival words of the one-launch layer kernel's exchange (windows of <= 16 rows): [2][world][R][H / 128]
    h->win_flag_bytes = R <= 16 ? ((size_t)2 * world * R * (H / 128) * 4 + 255) / 256 * 256 : 0;
    // {value, epoch} words of the flag-in-data exchange (windows of <= 16 rows): [2][world][R][H] x 8 bytes
    h->ll_bytes = R <= 16 ? (size_t)2 * world * R * H * 8 : 0;
    h->total_bytes = h->tail() + 256;
    if (cudaMalloc((void **)&h->local, h->total_bytes) != cudaSuccess || cudaMemset(h->local, 0, h->total_bytes) != cudaSuccess ||
        (!h->fin_bytes && cudaMalloc((void **)&h->out, R * H * 4) != cudaSuccess)) {
        glmflash_ep_free(h);
        return fail("cudaMalloc(ep buffers) failed");
    }
    if (h->fin_bytes) h->out = (float *)(h->local + h->recv_bytes + h->flag_bytes);
    h->peer_base[rank] = h->local;
    if (world == 1) h->connected = true;
    *out = h;
    return 0;
}

extern "C" void glmflash_ep_free(glmflash_ep *h) {
    if (!h) return;
    for (int k = 0; k < h->world; ++k)
        if (h->opened[k]) cudaIpcCloseMemHandle(h->peer_base[k]);
    if (!h->fin_bytes) cudaFree(h->out);
    cudaFree(h->local);
    delete h;
}

extern "C" int glmflash_ep_get_handle(glmflash_ep *h, void *handle_out) {
    GF_REQUIRE(h && handle_out, "null argument");
    EpBlob b{};
    GF_CUDA(cudaIpcGetMemHandle(&b.mem, h->local));
    b.config_hash = ep_config_hash(h->cfg, h->world, h->chunk_rows, h->use_ll);
    memcpy(handle_out, &b, sizeof(b));
    return 0;
}

extern "C" int glmflash_ep_connect(glmflash_ep *h, const void *all_handles) {
    GF_REQUIRE(h && all_handles, "null argument");
    GF_REQUIRE(!h->connected, "already connected");
    const unsigned char *p = (const unsigned char *)all_handles;
    const uint64_t mine = ep_config_hash(h->cfg, h->world, h->chunk_rows, h->use_ll);
    for (int k = 0; k < h->world; ++k) {                      // every rank's blob is checked before any mapping is made
        EpBlob b;
        memcpy(&b, p + (size_t)k * sizeof(b), sizeof(b));
        GF_REQUIRE(b.config_hash == mine, "rank " + std::to_string(k) + " was built with a different configuration "
                   "(hidden / inter / experts / slots / max_rows / world must agree on every rank)");
    }
    for (int k = 0; k < h->world; ++k) {
        if (k == h->rank) continue;
        EpBlob b;
        memcpy(&b, p + (size_t)k * sizeof(b), sizeof(b));
        const cudaIpcMemHandle_t m = b.mem;
        void *base = nullptr;
        GF_CUDA(cudaIpcOpenMemHandle(&base, m, cudaIpcMemLazyEnablePeerAccess));
        h->peer_base[k] = base;
        h->opened[k] = true;
    }
    h->connected = true;
    return 0;
}

extern "C" int glmflash_ep_combine(glmflash_ep *h, void *stream, const float *Y, const int32_t *picks, const float *route_w,
                                   int rows, int shared_here) {
    GF_REQUIRE(h && Y && picks && route_w, "null argument");
    GF_REQUIRE(h->connected, "glmflash_ep_connect has not been called");
    GF_REQUIRE(rows > 0 && rows <= h->cfg.max_rows, "rows outside the scratch bound");
    const glmflash_config &c = h->cfg;
    GF_REQUIRE(shared_here >= 0 && shared_here <= 2, "shared_here must be 0, 1 or 2");
    GF_REQUIRE(shared_here != 2 || (rows <= 16 && c.expert_hi > c.expert_lo && c.expert_lo % (c.expert_hi - c.expert_lo) == 0 &&
                                    (c.experts + c.expert_hi - c.expert_lo - 1) / (c.expert_hi - c.expert_lo) <= 32),
               "shared_here = 2 (owner decided per window) needs a window of <= 16 rows and equal expert windows of at most 32 ranks");
    EpPeers peers{};
    for (int k = 0; k < h->world; ++k) {
        peers.recv[k] = (float *)h->peer_base[k];
        peers.flags[k] = (unsigned *)((unsigned char *)h->peer_base[k] + h->recv_bytes);
        peers.fin[k] = (float *)((unsigned char *)h->peer_base[k] + h->recv_bytes + h->flag_bytes);
        peers.fin_flags[k] = (unsigned *)((unsigned char *)h->peer_base[k] + h->recv_bytes + h->flag_bytes + h->fin_bytes);
        peers.ll[k] = (uint2 *)((unsigned char *)h->peer_base[k] + h->ll_offset());
    }
    unsigned *epoch = (unsigned *)(h->local + h->tail());
    const dim3 grid((unsigned)((c.hidden / 4 + EP_THREADS - 1) / EP_THREADS), (unsigned)rows);
    if (rows > 16 && h->world > 1)
        return launch_k(h->bf16_rows ? ep_exchange_rows_kernel<true> : ep_exchange_rows_kernel<false>,
                        dim3((unsigned)((rows + h->chunk_rows - 1) / h->chunk_rows)), dim3(EP_THREADS), 0, (cudaStream_t)stream, c.pdl != 0,
                        Y, picks, route_w, h->out, peers, epoch, epoch + 1, (int *)(epoch + 2), h->rank, h->world, rows, c.max_rows,
                        h->max_ctas, c.slots, c.hidden, c.experts, shared_here, c.expert_lo, c.expert_hi, c.shared_row_lo,
                        c.shared_row_hi, h->wait_polls, h->chunk_rows);
    if (h->ll_bytes && h->use_ll)
        return launch_k(ep_combine_ll_kernel, grid, dim3(EP_THREADS), 0, (cudaStream_t)stream, c.pdl != 0, Y, picks, route_w, h->out,
                        peers, epoch, epoch + 1, (int *)(epoch + 2), h->rank, h->world, rows, c.max_rows, c.slots, c.hidden,
                        c.experts, shared_here, c.expert_lo, c.expert_hi, h->wait_polls);
    return launch_k(ep_combine_kernel, grid, dim3(EP_THREADS), 0, (cudaStream_t)stream, c.pdl != 0, Y, picks, route_w, h->out,
                    peers, epoch, epoch + 1, (int *)(epoch + 2), h->rank, h->world, rows, c.max_rows, h->max_ctas, c.slots,
                    c.hidden, c.experts, shared_here, c.expert_lo, c.expert_hi, c.shared_row_lo, c.shared_row_hi, h->wait_polls);
}

extern "C" int glmflash_ep_set_exchange_bf16(glmflash_ep *h, int on) {
    GF_REQUIRE(h != nullptr, "null argument");
    h->bf16_rows = on != 0;
    return 0;
}

extern "C" int glmflash_ep_set_wait_limit(glmflash_ep *h, uint32_t polls) {
    GF_REQUIRE(h != nullptr && polls > 0, "null argument or zero limit");
    h->wait_polls = polls;
    return 0;
}

// Single-process hosts (one process driving several GPUs with peer access enabled, or a test on one GPU): connect
// with raw device pointers to the peers' buffers instead of IPC handles.
extern "C" void *glmflash_ep_local_base(const glmflash_ep *h) { return h ? h->local : nullptr; }
extern "C" int glmflash_ep_connect_ptrs(glmflash_ep *h, void *const *peer_bases) {
    GF_REQUIRE(h && peer_bases, "null argument");
    GF_REQUIRE(!h->connected, "already connected");
    for (int k = 0; k < h->world; ++k) {
        if (k == h->rank) continue;
        GF_REQUIRE(peer_bases[k] != nullptr, "null peer buffer");
        h->peer_base[k] = peer_bases[k];
    }
    h->connected = true;
    return 0;
}

extern "C" float *glmflash_ep_output(const glmflash_ep *h) { return h ? h->out : nullptr; }
extern "C" const int32_t *glmflash_ep_status(const glmflash_ep *h) {
    return h ? (const int32_t *)(h->local + h->tail() + 8) : nullptr;
}
// After a peer time-out the status word stays set and every later wait gives up early, so that a dead peer costs one
// time-out and not one per block; the host clears it here when it has dealt with the failure.
extern "C" int glmflash_ep_clear_status(glmflash_ep *h, void *stream) {
    GF_REQUIRE(h != nullptr, "null argument");
    GF_CUDA(cudaMemsetAsync(h->local + h->tail() + 8, 0, 4, (cudaStream_t)stream));
    return 0;
}

namespace gf {
// The peer table of the one-launch layer kernel's exchange (window.cu).
int ep_window_peers(glmflash_ep *h, WinPeers *out, float **result) {
    GF_REQUIRE(h && out && result, "null argument");
    GF_REQUIRE(h->connected, "glmflash_ep_connect has not been called");
    GF_REQUIRE(h->win_flag_bytes > 0, "this exchange owner was built for more than 16 rows");
    *out = WinPeers{};
    for (int k = 0; k < h->world; ++k) {
        out->recv[k] = (float *)h->peer_base[k];
        out->flags[k] = (unsigned *)((unsigned char *)h->peer_base[k] + h->recv_bytes + h->flag_bytes + h->fin_bytes + h->fin_flag_bytes);
    }
    out->rank = h->rank; out->world = h->world; out->max_rows = h->cfg.max_rows; out->wait_polls = h->wait_polls;
    out->epoch = (unsigned *)(h->local + h->tail());
    out->status = (int *)(h->local + h->tail() + 8);
    *result = h->out;
    return 0;
}
}  // namespace gf
