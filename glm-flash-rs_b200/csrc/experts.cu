// ExpertGpu: the decode / verify owner (upstream src/experts.rs:365-563) and the single-linear probe.
#include <algorithm>
#include <new>

#include "gemv.cuh"
#include "owners.cuh"

namespace gf {
size_t experts_window_sync_words(const glmflash_config &c);

template <typename F>
static int set_smem(F *kernel, size_t bytes) {
    GF_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    return 0;
}

int launch_rot_in(cudaStream_t s, const void *x, bool x_is_bf16, int x_stride, const int *picks, const __half *suh0,
                  const __half *suh1, __half *out0, __half *out1, int K, int slots, int P, int mats, int E,
                  int shared_exl3, int e_lo, int e_hi, bool pdl) {
    const long items = (long)P * (K / 128) * mats;
    const unsigned grid = (unsigned)((items + 7) / 8);
    if (x_is_bf16)
        return launch_k(rot_in_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, pdl, (const __nv_bfloat16 *)x, x_stride,
                        picks, suh0, suh1, out0, out1, K, slots, P, mats, E, shared_exl3, e_lo, e_hi);
    return launch_k(rot_in_kernel<__half>, dim3(grid), dim3(256), 0, s, pdl, (const __half *)x, x_stride, picks, suh0, suh1,
                    out0, out1, K, slots, P, mats, E, shared_exl3, e_lo, e_hi);
}

int launch_gemv(cudaStream_t s, int mats, GemvArgs a, int umax, bool pdl) {
    const int sets = a.maxm > 8 ? 2 : 1;
    gemv_split(a.K, a.KTC, a.SK);
    GF_REQUIRE(a.SK * a.KTC == a.K / 16 && a.KTC % 8 == 0, "K cannot be cut into whole 128-k blocks per split");
    GF_REQUIRE(a.KTC <= 64, "K is too large for the decode path (at most 16 copy barriers per CTA)");
    const size_t smem = gemv_smem_bytes(mats, sets, a.KTC);
    GF_REQUIRE(smem <= 200 * 1024, "K is too large for the decode path's shared-memory staging");
    static size_t configured[64][4] = {};
    int dev = 0;
    GF_CUDA(cudaGetDevice(&dev));
    size_t &have = configured[dev & 63][(mats - 1) * 2 + (sets - 1)];
    if (have < smem) {                             // raise the dynamic shared-memory limit of this instantiation once
        if (mats == 2 && sets == 1) { if (set_smem(gemv_kernel<2, 1>, smem)) return -1; }
        else if (mats == 2) { if (set_smem(gemv_kernel<2, 2>, smem)) return -1; }
        else if (sets == 1) { if (set_smem(gemv_kernel<1, 1>, smem)) return -1; }
        else { if (set_smem(gemv_kernel<1, 2>, smem)) return -1; }
        have = smem;
    }
    const dim3 grid((unsigned)(a.N / 128), (unsigned)a.SK, (unsigned)umax), block(GEMV_THREADS), cluster(1, a.SK, 1);
    if (mats == 2 && sets == 1) return launch_kc(gemv_kernel<2, 1>, grid, block, cluster, smem, s, pdl, a);
    if (mats == 2) return launch_kc(gemv_kernel<2, 2>, grid, block, cluster, smem, s, pdl, a);
    if (sets == 1) return launch_kc(gemv_kernel<1, 1>, grid, block, cluster, smem, s, pdl, a);
    return launch_kc(gemv_kernel<1, 2>, grid, block, cluster, smem, s, pdl, a);
}

int check_config(const glmflash_config *cfg, size_t cfg_bytes, int max_rows_limit) {
    GF_REQUIRE(cfg != nullptr, "config is null");
    GF_REQUIRE(cfg_bytes == sizeof(glmflash_config), "config size mismatch (ABI)");
    GF_REQUIRE(cfg->hidden > 0 && cfg->hidden % 256 == 0, "hidden must be a positive multiple of 256");
    GF_REQUIRE(cfg->inter > 0 && cfg->inter % 256 == 0, "inter must be a positive multiple of 256");
    GF_REQUIRE(cfg->experts > 0 && cfg->experts < 1024, "experts must be in 1..1023");
    GF_REQUIRE(cfg->slots >= 2 && cfg->slots <= 32, "slots must be in 2..32");
    GF_REQUIRE(cfg->max_rows >= 1 && cfg->max_rows <= max_rows_limit, "max_rows outside the scratch bound");
    GF_REQUIRE(cfg->expert_lo >= 0 && cfg->expert_hi <= cfg->experts && cfg->expert_lo <= cfg->expert_hi,
               "expert window must satisfy 0 <= lo <= hi <= experts");
    GF_REQUIRE(cfg->limit > 0.f, "limit must be positive");
    GF_REQUIRE(cfg->shared_exl3 >= 0 && cfg->shared_exl3 <= 2, "shared_exl3 must be 0, 1 or 2");
    if (cfg->shared_exl3 == 2) {
        const int W = cfg->expert_hi - cfg->expert_lo;
        GF_REQUIRE(cfg->max_rows <= 16, "shared_exl3 = 2 (owner decided per window) is for handles of <= 16 rows");
        GF_REQUIRE(W > 0 && cfg->expert_lo % W == 0 && (cfg->experts + W - 1) / W <= 32,
                   "shared_exl3 = 2 needs equal contiguous expert windows (expert_lo a multiple of the window size, at most 32 ranks)");
    }
    GF_REQUIRE(cfg->shared_row_lo >= 0 && cfg->shared_row_lo <= cfg->shared_row_hi, "shared-expert row window must satisfy 0 <= lo <= hi");
    GF_REQUIRE(cfg->shared_row_hi == 0 || cfg->max_rows > 16, "a shared-expert row window needs a handle for more than 16 rows");
    int dev_count = 0;
    if (cudaGetDeviceCount(&dev_count) != cudaSuccess || dev_count == 0) return fail("no CUDA device: there is no CPU path");
    return 0;
}

}  // namespace gf

using namespace gf;

extern "C" int glmflash_experts_new(const glmflash_config *cfg, size_t cfg_bytes, glmflash_experts **out) {
    GF_REQUIRE(out != nullptr, "out is null");
    *out = nullptr;
    if (check_config(cfg, cfg_bytes, 16)) return -1;      // upstream: 1..=MAX_ROWS (16), src/experts.rs:391-394
    glmflash_experts *e = new (std::nothrow) glmflash_experts();
    GF_REQUIRE(e != nullptr, "out of host memory");
    e->cfg = *cfg;
    const size_t H = cfg->hidden, I = cfg->inter, P = (size_t)cfg->max_rows * cfg->slots;
    auto alloc = [&](void **p, size_t bytes) -> int {
        GF_CUDA(cudaMalloc(p, bytes));
        GF_CUDA(cudaMemset(*p, 0, bytes));
        return 0;
    };
    e->sync_words = experts_window_sync_words(*cfg);
    if (alloc((void **)&e->xg, P * H * 2) || alloc((void **)&e->xu, P * H * 2) || alloc((void **)&e->xd, P * I * 2) ||
        alloc((void **)&e->y, P * H * 4) || alloc((void **)&e->status, 4) ||
        alloc((void **)&e->z1, (size_t)2 * (H / 128) * P * I * 4) || alloc((void **)&e->z2, (size_t)(I / 128) * P * H * 4) ||
        alloc((void **)&e->sync, e->sync_words * 4) || alloc((void **)&e->out, (size_t)cfg->max_rows * H * 4)) {
        glmflash_experts_free(e);
        return -1;
    }
    *out = e;
    return 0;
}

extern "C" void glmflash_experts_free(glmflash_experts *e) {
    if (!e) return;
    cudaFree(e->xg); cudaFree(e->xu); cudaFree(e->xd); cudaFree(e->y); cudaFree(e->status);
    cudaFree(e->z1); cudaFree(e->z2); cudaFree(e->sync); cudaFree(e->out);
    delete e;
}

extern "C" int glmflash_experts_run_rows(glmflash_experts *e, void *stream, const glmflash_weights *w, const void *input,
                                         int x_stride, const int32_t *picks, const int32_t *ids, const int32_t *count,
                                         const int32_t *members, int rows, int maxm) {
    GF_REQUIRE(e && w && input && picks && ids && count && members, "null argument");
    const glmflash_config &c = e->cfg;
    GF_REQUIRE(c.shared_exl3 != 2, "shared_exl3 = 2 (owner decided per window) is served by the layer calls, not by run_rows");
    GF_REQUIRE(rows > 0 && rows <= c.max_rows && maxm >= rows && maxm <= c.max_rows, "expert verifier row/member bounds");
    GF_REQUIRE(x_stride >= c.hidden && x_stride % 4 == 0, "x_stride must be >= hidden and a multiple of 4");
    GF_REQUIRE(((uintptr_t)w->gt | (uintptr_t)w->ut | (uintptr_t)w->dt) % 16 == 0, "trellis tensors must be 16-byte aligned");
    GF_REQUIRE(((uintptr_t)input) % 8 == 0, "input must be 8-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    const bool pdl = c.pdl != 0;
    const int H = c.hidden, I = c.inter, P = rows * c.slots, E1 = c.experts + 1;
    const int umax = std::min(rows * (c.slots - 1) + 1, E1);
    if ((e->phases & 1) &&
        launch_rot_in(s, input, true, x_stride, picks, (const __half *)w->suh_g, (const __half *)w->suh_u, e->xg, e->xu, H,
                      c.slots, P, 2, c.experts, c.shared_exl3, c.expert_lo, c.expert_hi, pdl))
        return -1;
    GemvArgs a{};
    a.ids = ids; a.count = count; a.members = members;
    a.status = e->status;
    a.P = P; a.maxm = maxm; a.slots = c.slots; a.E = c.experts; a.e_lo = c.expert_lo; a.e_hi = c.expert_hi;
    a.shared_exl3 = c.shared_exl3; a.limit = c.limit;
    // gate + up, SwiGLU, down-input rotation -> xd
    a.X0 = e->xg; a.X1 = e->xu; a.T0 = w->gt; a.T1 = w->ut;
    a.sv0 = (const __half *)w->svh_g; a.sv1 = (const __half *)w->svh_u; a.sd = (const __half *)w->suh_d;
    a.xd = e->xd; a.y = nullptr; a.K = H; a.N = I; a.mode = GEMV_GATEUP;
    if ((e->phases & 2) && launch_gemv(s, 2, a, umax, pdl)) return -1;
    if (!(e->phases & 4)) return 0;
    // down -> y
    a.X0 = e->xd; a.X1 = e->xd; a.T0 = w->dt; a.T1 = w->dt;
    a.sv0 = (const __half *)w->svh_d; a.sv1 = nullptr; a.sd = nullptr;
    a.xd = nullptr; a.y = e->y; a.K = I; a.N = H; a.mode = GEMV_DOWN;
    return launch_gemv(s, 1, a, umax, pdl);
}

// The layer pipeline's form of run_rows (used by Moe for windows of <= 16 rows): no grouping tables and no rotation
// kernel -- the gate/up kernel derives expert and members from the routing table and rotates the input itself, the
// down kernel derives them again.  Two launches instead of four; the arithmetic per pair is that of run_rows.
namespace gf {
int experts_run_fused(glmflash_experts *e, cudaStream_t s, const glmflash_weights *w, const void *input, int x_stride,
                      const int32_t *picks, int rows) {
    const glmflash_config &c = e->cfg;
    GF_REQUIRE(rows > 0 && rows <= c.max_rows, "expert verifier row/member bounds");
    GF_REQUIRE(x_stride >= c.hidden && x_stride % 4 == 0, "x_stride must be >= hidden and a multiple of 4");
    GF_REQUIRE(((uintptr_t)w->gt | (uintptr_t)w->ut | (uintptr_t)w->dt) % 16 == 0, "trellis tensors must be 16-byte aligned");
    GF_REQUIRE(((uintptr_t)input | (uintptr_t)w->suh_g | (uintptr_t)w->suh_u) % 8 == 0, "input and scale vectors must be 8-byte aligned");
    const bool pdl = c.pdl != 0;
    const int H = c.hidden, I = c.inter, P = rows * c.slots, E1 = c.experts + 1;
    // clusters per column block: the distinct experts of the window that THIS GPU computes, at most its expert window
    // (+ the shared expert) -- an expert-parallel rank does not launch CTAs for the other ranks' experts
    const int mine = (c.expert_hi - c.expert_lo) + (c.shared_exl3 ? 1 : 0);
    const int umax = std::max(1, std::min(std::min(rows * (c.slots - 1) + 1, E1), mine));
    GemvArgs a{};
    a.status = e->status;
    a.P = P; a.maxm = rows; a.slots = c.slots; a.E = c.experts; a.e_lo = c.expert_lo; a.e_hi = c.expert_hi;
    a.shared_exl3 = c.shared_exl3; a.limit = c.limit;
    a.picks = picks; a.rows = rows;
    // gate + up on the rotated input, SwiGLU, down-input rotation -> xd
    a.xin = (const __nv_bfloat16 *)input; a.x_stride = x_stride; a.wait_first = 1;
    a.suh0 = (const __half *)w->suh_g; a.suh1 = (const __half *)w->suh_u;
    a.T0 = w->gt; a.T1 = w->ut;
    a.sv0 = (const __half *)w->svh_g; a.sv1 = (const __half *)w->svh_u; a.sd = (const __half *)w->suh_d;
    a.xd = e->xd; a.y = nullptr; a.K = H; a.N = I; a.mode = GEMV_GATEUP;
    // down -> y
    GemvArgs d = a;
    d.xin = nullptr; d.wait_first = 0; d.suh0 = d.suh1 = nullptr;
    d.X0 = e->xd; d.X1 = e->xd; d.T0 = w->dt; d.T1 = w->dt;
    d.sv0 = (const __half *)w->svh_d; d.sv1 = nullptr; d.sd = nullptr;
    d.xd = nullptr; d.y = e->y; d.K = I; d.N = H; d.mode = GEMV_DOWN;
    if ((e->phases & 2) && launch_gemv(s, 2, a, umax, pdl)) return -1;
    if (!(e->phases & 4)) return 0;
    // (the routing table was consumed by the kernel before: the down kernel may read it before its dependency wait)
    return launch_gemv(s, 1, d, umax, pdl);
}
}  // namespace gf

extern "C" int glmflash_experts_set_phases(glmflash_experts *e, int mask) {
    GF_REQUIRE(e != nullptr, "null argument");
    e->phases = mask;
    return 0;
}

extern "C" float *glmflash_experts_y(const glmflash_experts *e) { return e ? e->y : nullptr; }
extern "C" const uint16_t *glmflash_experts_xd(const glmflash_experts *e) { return e ? (const uint16_t *)e->xd : nullptr; }
extern "C" const int32_t *glmflash_experts_status(const glmflash_experts *e) { return e ? e->status : nullptr; }
extern "C" int glmflash_experts_clear_status(glmflash_experts *e, void *stream) {
    GF_REQUIRE(e != nullptr, "null argument");
    // a give-up may have left arrival counters of the one-launch kernel half way: clear them with the status word
    GF_CUDA(cudaMemsetAsync(e->status, 0, 4, (cudaStream_t)stream));
    GF_CUDA(cudaMemsetAsync(e->sync, 0, e->sync_words * 4, (cudaStream_t)stream));
    return 0;
}

// ---- single EXL3 linear (fp16 in, fp16 out): rot_in + one-matrix GEMV with the fp16 epilogue ---------------
namespace {
struct LinearScratch {
    size_t xr, tables, total;
};
LinearScratch linear_layout(int K, int N) {
    (void)N;
    LinearScratch L;
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += (bytes + 255) / 256 * 256; return o; };
    L.xr = take((size_t)16 * K * 2);                // rotated input rows
    L.tables = take((size_t)(2 + 16) * 4 + 4);      // ids[1], count[1], members[16], status
    L.total = off;
    return L;
}
__global__ void linear_tables_kernel(int *tables, int rows) {
    // ids[0] = 0, count = 1, members[m] = m * 32 (row m, slot 0) for m < rows, else -1; status = 0
    const int t = threadIdx.x;
    if (t == 0) { tables[0] = 0; tables[1] = 1; tables[18] = 0; }
    if (t < 16) tables[2 + t] = t < rows ? t * 32 : -1;
}
}  // namespace

extern "C" size_t glmflash_exl3_linear_scratch_bytes(int K, int N) {
    if (K <= 0 || N <= 0 || K % 256 || N % 128) return 0;
    return linear_layout(K, N).total;
}

extern "C" int glmflash_exl3_linear(void *stream, const uint16_t *x, int rows, const uint32_t *words, const uint16_t *suh,
                                    const uint16_t *svh, int K, int N, uint16_t *y, void *scratch) {
    GF_REQUIRE(x && words && suh && svh && y && scratch, "null argument");
    GF_REQUIRE(K > 0 && K % 256 == 0 && N > 0 && N % 128 == 0, "K must be a multiple of 256 and N of 128");
    GF_REQUIRE(rows >= 1 && rows <= 16, "rows must be in 1..16");
    GF_REQUIRE(((uintptr_t)words) % 16 == 0 && ((uintptr_t)scratch) % 256 == 0, "words 16-byte, scratch 256-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    const LinearScratch L = linear_layout(K, N);
    unsigned char *base = (unsigned char *)scratch;
    int *tables = (int *)(base + L.tables);
    linear_tables_kernel<<<1, 32, 0, s>>>(tables, rows);
    GF_CUDA(cudaGetLastError());
    __half *xr = (__half *)(base + L.xr);
    if (launch_rot_in(s, x, false, K, nullptr, (const __half *)suh, (const __half *)suh, xr, xr, K, 1, rows, 1, 1, 1, 0, 2, false))
        return -1;
    GemvArgs a{};
    a.X0 = xr; a.X1 = xr; a.T0 = words; a.T1 = words;
    a.ids = tables; a.count = tables + 1; a.members = tables + 2;
    a.status = tables + 18;
    a.sv0 = (const __half *)svh; a.xd = (__half *)y;
    a.K = K; a.N = N; a.P = rows; a.maxm = rows; a.slots = 1; a.E = 1; a.e_lo = 0; a.e_hi = 1;
    a.shared_exl3 = 1; a.mode = GEMV_LINEAR; a.limit = 10.f;
    return launch_gemv(s, 1, a, 1, false);
}

// ---- the single EXL3 linear for callers that must not allocate ------------------------------------------------
// Same computation as glmflash_exl3_linear, but the scratch lives in a fixed array inside the library image instead
// of caller-provided memory.  It is meant for hosts that own the whole device heap themselves (upstream's Rust
// `Device` hands out every byte of device memory at start-up and keeps the request path free of allocator calls),
// and for latency-critical loops in which a cudaMalloc/cudaFree would serialise the device behind the allocator.
// The array is part of every loaded copy of the library: each GPU that loads it holds these bytes until exit.
namespace {
constexpr int STATIC_LINEAR_MAX_K = 4096;
constexpr size_t STATIC_LINEAR_BYTES = 135168;            // 132 KiB >= linear_layout(4096, N).total
static __device__ __align__(256) unsigned char g_static_linear_scratch[STATIC_LINEAR_BYTES];
void *g_static_linear_ptr[64] = {};                       // device address of the array, per device ordinal
}  // namespace

extern "C" size_t glmflash_exl3_linear_static_max_bytes(void) { return STATIC_LINEAR_BYTES; }

extern "C" int glmflash_exl3_linear_static(void *stream, const uint16_t *x, int rows, const uint32_t *words,
                                           const uint16_t *suh, const uint16_t *svh, int K, int N, uint16_t *y) {
    GF_REQUIRE(K > 0 && K % 256 == 0 && N > 0 && N % 128 == 0, "K must be a multiple of 256 and N of 128");
    GF_REQUIRE(K <= STATIC_LINEAR_MAX_K,
               "shape exceeds the built-in scratch (K <= 4096): use glmflash_exl3_linear with caller scratch");
    GF_REQUIRE(linear_layout(K, N).total <= STATIC_LINEAR_BYTES, "shape exceeds the built-in scratch");
    int dev = 0;
    GF_CUDA(cudaGetDevice(&dev));
    GF_REQUIRE(dev >= 0 && dev < 64, "device ordinal out of range");
    if (!g_static_linear_ptr[dev]) {
        // In host code the array's name is only a handle; the address a kernel can use comes from the runtime,
        // once per device, with that device current.
        void *p = nullptr;
        GF_CUDA(cudaGetSymbolAddress(&p, g_static_linear_scratch));
        GF_REQUIRE(p != nullptr, "cudaGetSymbolAddress returned a null address");
        g_static_linear_ptr[dev] = p;
    }
    return glmflash_exl3_linear(stream, x, rows, words, suh, svh, K, N, y, g_static_linear_ptr[dev]);
}

#ifdef GF_TRACE
extern "C" int glmflash_trace_set(long long *buffer) {
    GF_CUDA(cudaMemcpyToSymbol(gf::g_trace, &buffer, sizeof(buffer)));
    return 0;
}
#endif
