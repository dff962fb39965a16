// Shared device helpers of the B200 EXL3 expert path: the trellis codebook, the 128-point Hadamard
// transform, rounding helpers, TMA bulk copies with bounded mbarrier waits, and host-side error plumbing.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string.h>

#include <string>

#include "../../include/glmflash_b200.h"

namespace gf {

constexpr float HAD_SCALE = 0.08838834764831845f;  // 1 / sqrt(128)
constexpr uint32_t MCG_MUL = 0xCBAC1FEDu;
constexpr uint32_t MCG_AND = 0x8FFF8FFFu;
constexpr uint32_t MCG_XOR = 0x3B603B60u;

// ---- host-side error plumbing --------------------------------------------------------------------------
std::string &last_error();
int fail(const std::string &msg);
int fail_cuda(cudaError_t e, const char *what);
#define GF_CUDA(call)                                             \
    do {                                                          \
        cudaError_t gf_e_ = (call);                               \
        if (gf_e_ != cudaSuccess) return gf::fail_cuda(gf_e_, #call); \
    } while (0)
#define GF_REQUIRE(cond, msg)                \
    do {                                     \
        if (!(cond)) return gf::fail(msg);   \
    } while (0)

// Launch with or without the programmatic-dependent-launch attribute (the kernel's griddepcontrol instructions
// are no-ops without it).
template <typename... KArgs, typename... Args>
int launch_kc(void (*kernel)(KArgs...), dim3 grid, dim3 block, dim3 cluster, size_t smem, cudaStream_t s, bool pdl,
              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[3];
    int n = 0;
    if (pdl) {
        at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster.x * cluster.y * cluster.z > 1) {
        at[n].id = cudaLaunchAttributeClusterDimension;
        at[n].val.clusterDim.x = cluster.x;
        at[n].val.clusterDim.y = cluster.y;
        at[n].val.clusterDim.z = cluster.z;
        ++n;
        // let the hardware balance the CTAs of a cluster over the SMs (measured a little faster than the default)
        at[n].id = cudaLaunchAttributeClusterSchedulingPolicyPreference;
        at[n].val.clusterSchedulingPolicyPreference = cudaClusterSchedulingPolicyLoadBalancing;
        ++n;
    }
    cfg.attrs = n ? at : nullptr;
    cfg.numAttrs = n;
    GF_CUDA(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
    return 0;
}
template <typename... KArgs, typename... Args>
int launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool pdl, Args... args) {
    return launch_kc(kernel, grid, block, dim3(1, 1, 1), smem, s, pdl, args...);
}

// ---- codebook ------------------------------------------------------------------------------------------
// The 32-bit codeword of a 16-bit trellis state: two fp16 halves whose sum is the weight
// (upstream native/exl3.cu:21-25).
__device__ __forceinline__ uint32_t codeword(uint32_t state) { return ((state * MCG_MUL) & MCG_AND) ^ MCG_XOR; }

// The weight itself: half-precision sum of the two halves, round to nearest even (upstream :26-29).
__device__ __forceinline__ __half codebook(uint32_t state) {
    const uint32_t x = codeword(state);
    return __hadd(__ushort_as_half((unsigned short)(x & 0xffffu)), __ushort_as_half((unsigned short)(x >> 16)));
}

// Codewords of the two states packed in u = (state_hi << 16) | state_lo.
// GF_MCG_MAD = 1 trades two ALU operations (mask, shift) for one multiply-add:
//   (u & 0xffff) * C  ==  u * C - (((u >> 16) * C) << 16)   (mod 2^32),
// because the integer-multiply pipe has slack while the ALU pipe is the bottleneck of the GEMV.
#ifndef GF_MCG_MAD
#define GF_MCG_MAD 1
#endif
__device__ __forceinline__ void codeword_pair(uint32_t u, uint32_t &x_hi, uint32_t &x_lo) {
    const uint32_t h = u >> 16;
#if GF_MCG_MAD
    uint32_t ph, pu, pl;
    asm("mul.lo.u32 %0, %1, %2;" : "=r"(ph) : "r"(h), "r"(MCG_MUL));
    asm("mul.lo.u32 %0, %1, %2;" : "=r"(pu) : "r"(u), "r"(MCG_MUL));
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(pl) : "r"(ph), "r"(0xFFFF0000u), "r"(pu));
    x_hi = (ph & MCG_AND) ^ MCG_XOR;
    x_lo = (pl & MCG_AND) ^ MCG_XOR;
#else
    x_hi = codeword(h);
    x_lo = codeword(u & 0xffffu);
#endif
}

// ---- rounding helpers (the rounding points of upstream's epilogues, native/exl3.cu:243) ------------------
__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// ---- Hadamard ------------------------------------------------------------------------------------------
// 128 values held 4 per lane (lane L: values 4L..4L+3), natural order; butterflies stride 1, 2 in
// registers, 4..64 across lanes, each (lower + upper, lower - upper): upstream's order
// (native/exl3.cu:208-219 <=> src/experts.rs:25-42), so sums associate identically.
__device__ __forceinline__ void fwht128(float (&v)[4], int lane) {
    const float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
    v[0] = a + c; v[1] = b + d; v[2] = a - c; v[3] = b - d;
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float o = __shfl_xor_sync(0xffffffffu, v[j], m);
            v[j] = (lane & m) ? o - v[j] : v[j] + o;
        }
    }
}

// ---- the shared expert's owner, decided per window (config shared_exl3 == 2) -------------------------------
// Expert-parallel ranks hold contiguous windows of W routed experts (rank = id / W).  When the shared expert's owner is
// left to the device, it is the rank whose window holds the FEWEST distinct routed experts of the window's routing
// table (ties: the lowest rank): the rank that would otherwise idle longest takes the expert every row uses.  Every rank
// evaluates this on the same table, so all agree without an exchange, and the expert kernels and the combine /
// exchange kernels of a rank agree with each other.  At most 32 ranks (one lane each).
// `used`: bitmap (shared memory, 32 words) of the ids the table names.  Called by a whole warp; same result in every lane.
__device__ __forceinline__ int shared_owner_rank(const uint32_t *used, int E, int W, int lane) {
    const int G = (E + W - 1) / W;
    int c = 1023;
    if (lane < G) {
        c = 0;
        for (int e = lane * W; e < min(E, (lane + 1) * W); ++e) c += (used[e >> 5] >> (e & 31)) & 1u;
    }
    int best = c * 32 + lane;
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, d));
    return best & 31;
}
// Block-level form for kernels that have no bitmap of their own: builds it from the routing table (np = rows x slots
// entries) in `used` (32 words of shared memory) and returns the owner rank in every thread.  All threads of the block call.
__device__ __forceinline__ int shared_owner_of_window(const int *picks, int np, int E, int W, uint32_t *used) {
    if (threadIdx.x < 32) used[threadIdx.x] = 0u;
    __syncthreads();
    for (int i = threadIdx.x; i < np; i += blockDim.x) {
        const int pk = picks[i];
        if (pk >= 0 && pk < E) atomicOr(&used[pk >> 5], 1u << (pk & 31));
    }
    __syncthreads();
    return shared_owner_rank(used, E, W, threadIdx.x & 31);
}

// ---- shared-memory addressing, TMA bulk copy, mbarrier -----------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// The same with a suspend-time hint: the thread may sleep up to `ns` nanoseconds inside the instruction (it
// returns at once when the phase completes), so a waiting warp does not compete for issue slots.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t *bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls and reports false (the caller records an error status and
// leaves); nothing in this library spins without a bound.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, const int *status = nullptr, uint32_t limit = 4000000u) {
    if (mbar_try_wait(bar, parity)) return true;
    for (uint32_t i = 0; i < limit; ++i) {            // the waiting thread may sleep inside the instruction: no issue slots taken
        if (mbar_try_wait_hint(bar, parity, 400u)) return true;
        // a wait of this launch has already given up (the status word is set): do not sit out the limit in every CTA
        if (status && (i & 255u) == 255u && *reinterpret_cast<const volatile int *>(status) != 0) return false;
    }
    return false;
}
// 1-D TMA bulk copy global -> shared, completion counted in bytes on an mbarrier.  Both addresses and the
// size are multiples of 16 bytes.
__device__ __forceinline__ void tma_load_1d(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Thread-block cluster: barrier over all threads of the cluster, and the address of a peer CTA's copy of a shared
// memory object (distributed shared memory).  A cluster of one CTA is its own peer.
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
template <typename Tp>
__device__ __forceinline__ const Tp *cluster_map(const Tp *p, uint32_t rank) {
    uint64_t out;
    asm volatile("mapa.u64 %0, %1, %2;" : "=l"(out) : "l"((uint64_t)p), "r"(rank));
    return reinterpret_cast<const Tp *>(out);
}

// Programmatic dependent launch: let the next kernel of the stream start its prologue; wait until the
// previous kernel's results are visible.  Both are no-ops for a kernel launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Device status word shared by kernels with bounded waits: 0 = fine, otherwise the first failure code.
enum : int { GF_STATUS_OK = 0, GF_STATUS_TMA_TIMEOUT = 1, GF_STATUS_TMEM = 2, GF_STATUS_MMA_TIMEOUT = 3, GF_STATUS_PEER_TIMEOUT = 4 };

}  // namespace gf
