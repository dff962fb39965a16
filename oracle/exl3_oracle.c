/*
 * CPU oracle for the EXL3 (trellis, 4 bits per weight) MoE expert path.  TEST INFRASTRUCTURE ONLY:
 * the shipped library never links, loads or calls this file; tests and the benchmark's CPU-baseline
 * leg use it as the checker and as the timed host-core baseline.
 *
 * It restates, in plain C, the scalar algorithm of the reference (cuylerstuwe/glm-flash-rs):
 *   codebook            src/experts.rs:43-46        (device form native/exl3.cu:21-30)
 *   tile unpack         src/experts.rs:47-74        (device form native/exl3.cu:33-40)
 *   Hadamard            src/experts.rs:25-42        (device form native/exl3.cu:208-219)
 *   bf16 / fp16 round   src/experts.rs:19-24
 *   matmul order        src/experts.rs:76-96
 *   one-expert pipeline src/experts.rs:100-135  <=> native/exl3.cu:224-321
 *   pair / member codes native/exl3.cu:160-166,228-231
 *   grouping contract   native/grouping.cu:67-100, src/grouping.rs:143-192
 *   combine             src/moe.rs:171-181 (call site; the kernel's source is absent upstream)
 *   router, top-k       src/moe.rs:77-111 (call sites; sources absent upstream: the benchmark's definition, PARITY UNPINNED)
 *
 * Pinning: the reference's own known-answer tests for this path are hadamard_involution and
 * codebook_finite (src/experts.rs:566-583); both are reproduced in tests/.  The reference holds no
 * golden vectors for expert outputs; tests/golden/ref_sm100.npz holds outputs of the reference's own
 * CUDA kernels (compiled unmodified for sm_100a, run on a B200 by tests/golden/make_golden.py): its
 * trellis decode, its decode-path and prefill-path layer results and its grouping.  tests/test_golden.py
 * checks this oracle against them on the CPU (decode and grouping bit-exact), and the GPU tests compare
 * the oracle with the same kernels live (oracle/_ref).
 *
 * Build: make -C oracle   (gcc -O2 -fopenmp -ffp-contract=off; contraction is off so that the
 * fp32 accumulation is mul-then-add exactly as the reference's scalar Rust).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define HAD_SCALE 0.088388346f /* src/experts.rs:11 (f32 nearest to 1/sqrt(128)) */

/* ---------------------------------------------------------------- number formats */

static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* IEEE binary16 -> binary32, exact. */
float gfo_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ff;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        float v = (float)man * 5.9604644775390625e-08f; /* 2^-24 */
        return sign ? -v : v;
    }
    if (exp == 31) return bits_f32(sign | 0x7f800000u | (man << 13));
    return bits_f32(sign | ((exp + 112) << 23) | (man << 13));
}

/* binary64 -> binary16, round to nearest even (one rounding from the exact double). */
static uint16_t f64_to_f16(double d) {
    uint64_t u; memcpy(&u, &d, 8);
    uint16_t sign = (uint16_t)((u >> 48) & 0x8000u);
    double a = fabs(d);
    if (isnan(d)) return (uint16_t)(sign | 0x7e00u);
    if (a >= 65520.0) return (uint16_t)(sign | 0x7c00u);   /* rounds to inf */
    if (a < 6.103515625e-05) {                             /* below the smallest normal: subnormal grid 2^-24 */
        double q = a * 16777216.0;                          /* exact scaling */
        double r = nearbyint(q);                            /* default mode: ties to even */
        return (uint16_t)(sign | (uint16_t)r);              /* r == 1024 gives the smallest normal */
    }
    int e; double m = frexp(a, &e);                         /* a = m * 2^e, m in [0.5,1) */
    double q = ldexp(m, 11);                                /* in [1024, 2048) */
    double r = nearbyint(q);
    int ex = e - 1;                                         /* unbiased exponent of a */
    if (r >= 2048.0) { r = 1024.0; ex += 1; }
    return (uint16_t)(sign | (uint16_t)((ex + 15) << 10) | ((uint16_t)r & 0x3ff));
}
uint16_t gfo_f32_to_f16(float f) { return f64_to_f16((double)f); }

/* fp32 -> value of the nearest fp16 (src/experts.rs:22-24, hf). */
float gfo_hf(float x) { return gfo_f16_to_f32(gfo_f32_to_f16(x)); }

/* fp32 -> value of the nearest bf16, the reference's integer formula (src/experts.rs:19-21, bf). */
float gfo_bf(float x) {
    uint32_t b = f32_bits(x);
    return bits_f32((b + 0x7fffu + ((b >> 16) & 1u)) & 0xffff0000u);
}
uint16_t gfo_f32_to_bf16(float x) { return (uint16_t)(f32_bits(gfo_bf(x)) >> 16); }
float gfo_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* ---------------------------------------------------------------- codebook and tiles */

/* The "mcg" codebook: 16-bit state -> fp16 (bits).  src/experts.rs:43-46; native/exl3.cu:21-30 adds
 * the two halves with a half-precision add (round to nearest even), restated here exactly: the sum
 * of two binary16 values is exact in binary64, then rounded once. */
uint16_t gfo_codebook(uint32_t s) {
    uint32_t x = ((s * 0xCBAC1FEDu) & 0x8FFF8FFFu) ^ 0x3B603B60u;
    double lo = (double)gfo_f16_to_f32((uint16_t)(x & 0xffffu));
    double hi = (double)gfo_f16_to_f32((uint16_t)(x >> 16));
    return f64_to_f16(lo + hi);
}

/* The raw 32-bit codeword (two fp16 halves whose sum is the weight) of a state. */
uint32_t gfo_codeword(uint32_t s) { return ((s * 0xCBAC1FEDu) & 0x8FFF8FFFu) ^ 0x3B603B60u; }

/* Position p (0..255) of a tile -> (row k, column n) inside the 16x16 tile.  src/experts.rs:65-68. */
static inline void tile_pos(int p, int *row, int *col) {
    int lane = p / 8, j = p % 8;
    *row = 2 * (lane % 4) + (j & 1) + 8 * ((j >> 1) & 1);
    *col = lane / 4 + 8 * (j >> 2);
}

/* Bitstream form (src/experts.rs:58-69): the tile is a 1024-bit MSB-first circular stream, weight p
 * has the 16-bit state ending at bit 4p+4.  out[row*16+col] = fp16 bits. */
void gfo_decode_tile_stream(const uint32_t *tile, uint16_t *out) {
    for (int p = 0; p < 256; ++p) {
        int first = p * 4 + 4 + 1024 - 16, last = first + 16;
        int i0 = (first / 32) % 32, i1 = ((last - 1) / 32) % 32;
        int shift = ((last - 1) / 32 + 1) * 32 - last;
        uint64_t v = ((uint64_t)tile[i0] << 32) | (uint64_t)tile[i1];
        uint32_t state = (uint32_t)((v >> shift) & 0xffffu);
        int row, col; tile_pos(p, &row, &col);
        out[row * 16 + col] = gfo_codebook(state);
    }
}

/* Lane form (native/exl3.cu:33-40): lane L takes word L and word L-1 (circular), shifts the pair
 * right by 20 and cuts eight overlapping 16-bit states.  Must equal the bitstream form. */
void gfo_decode_tile_lanes(const uint32_t *tile, uint16_t *out) {
    for (int lane = 0; lane < 32; ++lane) {
        uint32_t w = tile[lane], p = tile[(lane + 31) & 31];
        uint32_t s = (uint32_t)((((uint64_t)p << 32) | w) >> 20);
        uint32_t st[8] = {(s >> 8) & 0xffffu, (s >> 4) & 0xffffu, s & 0xffffu, w >> 16,
                          (w >> 12) & 0xffffu, (w >> 8) & 0xffffu, (w >> 4) & 0xffffu, w & 0xffffu};
        for (int j = 0; j < 8; ++j) {
            int row, col; tile_pos(lane * 8 + j, &row, &col);
            out[row * 16 + col] = gfo_codebook(st[j]);
        }
    }
}

/* The 16-bit states of a tile in position order (for tests of kernels that keep states). */
void gfo_tile_states(const uint32_t *tile, uint16_t *states) {
    for (int p = 0; p < 256; ++p) {
        int first = p * 4 + 4 + 1024 - 16, last = first + 16;
        int i0 = (first / 32) % 32, i1 = ((last - 1) / 32) % 32;
        int shift = ((last - 1) / 32 + 1) * 32 - last;
        uint64_t v = ((uint64_t)tile[i0] << 32) | (uint64_t)tile[i1];
        states[p] = (uint16_t)((v >> shift) & 0xffffu);
    }
}

/* Whole matrix: words[K/16][N/16][32] -> w[K][N] as fp16 bits (src/experts.rs:47-74). */
void gfo_unpack_f16(const uint32_t *words, int K, int N, uint16_t *w) {
    int KT = K / 16, NT = N / 16;
#pragma omp parallel for schedule(static)
    for (int kt = 0; kt < KT; ++kt) {
        uint16_t t[256];
        for (int nt = 0; nt < NT; ++nt) {
            gfo_decode_tile_stream(words + ((size_t)kt * NT + nt) * 32, t);
            for (int r = 0; r < 16; ++r)
                memcpy(w + ((size_t)kt * 16 + r) * N + nt * 16, t + r * 16, 32);
        }
    }
}

/* Same, as fp32 values. threads = 1 keeps it single-threaded for the faithful timing. */
static void unpack_f32(const uint32_t *words, int K, int N, float *w, int threads) {
    int KT = K / 16, NT = N / 16;
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int kt = 0; kt < KT; ++kt) {
        uint16_t t[256];
        for (int nt = 0; nt < NT; ++nt) {
            gfo_decode_tile_stream(words + ((size_t)kt * NT + nt) * 32, t);
            for (int r = 0; r < 16; ++r)
                for (int c = 0; c < 16; ++c)
                    w[((size_t)kt * 16 + r) * N + nt * 16 + c] = gfo_f16_to_f32(t[r * 16 + c]);
        }
    }
}
void gfo_unpack_f32(const uint32_t *words, int K, int N, float *w) { unpack_f32(words, K, N, w, 1); }

/* ---------------------------------------------------------------- Hadamard */

/* Unnormalised Sylvester Walsh-Hadamard over each block of 128, strides 1..64, (a+b, a-b).
 * src/experts.rs:25-42.  n must be a multiple of 128. */
void gfo_had128(float *y, int n) {
    for (int b = 0; b + 128 <= n; b += 128) {
        float *blk = y + b;
        for (int stride = 1; stride < 128; stride *= 2)
            for (int base = 0; base < 128; base += stride * 2)
                for (int j = 0; j < stride; ++j) {
                    float a = blk[base + j], c = blk[base + j + stride];
                    blk[base + j] = a + c;
                    blk[base + j + stride] = a - c;
                }
    }
}

/* ---------------------------------------------------------------- matmul */

/* y[N] = x[K] @ w[K][N].
 * mode 0: the reference's order (src/experts.rs:76-96): K cut into sk splits x 4 "warps", each a
 *         left-to-right fp32 chain of separate multiply and add, warps added ((0+1)+2)+3, splits in
 *         ascending order.
 * mode 1: binary64 accumulation, rounded once to fp32 ("exact" target for error measurements). */
void gfo_matmul(const float *x, const float *w, int K, int N, int sk, int mode, float *y) {
    if (mode == 1) {
        double *acc = (double *)calloc((size_t)N, sizeof(double));
        for (int k = 0; k < K; ++k) {
            double xv = x[k];
            const float *wr = w + (size_t)k * N;
            for (int n = 0; n < N; ++n) acc[n] += xv * (double)wr[n];
        }
        for (int n = 0; n < N; ++n) y[n] = (float)acc[n];
        free(acc);
        return;
    }
    float *part = (float *)malloc((size_t)4 * N * sizeof(float));
    for (int n = 0; n < N; ++n) y[n] = 0.f;
    for (int split = 0; split < sk; ++split) {
        memset(part, 0, (size_t)4 * N * sizeof(float));
        for (int warp = 0; warp < 4; ++warp) {
            int begin = (split * 4 + warp) * K / (sk * 4), end = begin + K / (sk * 4);
            float *acc = part + (size_t)warp * N;
            for (int j = begin; j < end; ++j) {
                float xv = x[j];
                const float *wr = w + (size_t)j * N;
                for (int n = 0; n < N; ++n) acc[n] += xv * wr[n];
            }
        }
        for (int n = 0; n < N; ++n) {
            float partial = ((part[n] + part[N + n]) + part[2 * N + n]) + part[3 * N + n];
            y[n] += partial;
        }
    }
    free(part);
}

/* ---------------------------------------------------------------- EXL3 linear and expert */

/* Input rotation of one row: out[k] = hf(H(x * suh)[k] * HAD_SCALE).  src/experts.rs:105-106,
 * native/exl3.cu:224-241.  x already holds the activation values as fp32. */
static void rot_in(const float *x, const uint16_t *suh, int K, float *out) {
    for (int k = 0; k < K; ++k) out[k] = x[k] * gfo_f16_to_f32(suh[k]);
    gfo_had128(out, K);
    for (int k = 0; k < K; ++k) out[k] = gfo_hf(out[k] * HAD_SCALE);
}

/* One EXL3 linear on fp16 inputs: y = fp16( H( rot_in(x) @ W ) * HAD_SCALE * svh ).
 * x[rows][K] fp16 bits, words[K/16][N/16][32], suh[K], svh[N] fp16 bits, y[rows][N] fp16 bits.
 * (The single-matrix building block of src/experts.rs:100-135 with an fp16 output.) */
void gfo_linear_f16(const uint16_t *x, int rows, const uint32_t *words, const uint16_t *suh,
                    const uint16_t *svh, int K, int N, int sk, int mode, uint16_t *y, float *y32) {
    float *w = (float *)malloc((size_t)K * N * sizeof(float));
    unpack_f32(words, K, N, w, 0 + 1);
    float *xr = (float *)malloc((size_t)K * sizeof(float));
    float *rot = (float *)malloc((size_t)K * sizeof(float));
    float *acc = (float *)malloc((size_t)N * sizeof(float));
    for (int r = 0; r < rows; ++r) {
        for (int k = 0; k < K; ++k) xr[k] = gfo_f16_to_f32(x[(size_t)r * K + k]);
        rot_in(xr, suh, K, rot);
        gfo_matmul(rot, w, K, N, sk, mode, acc);
        gfo_had128(acc, N);
        for (int n = 0; n < N; ++n) {
            float v = acc[n] * HAD_SCALE * gfo_f16_to_f32(svh[n]);
            if (y32) y32[(size_t)r * N + n] = v;
            if (y) y[(size_t)r * N + n] = gfo_f32_to_f16(v);
        }
    }
    free(w); free(xr); free(rot); free(acc);
}

/* The nine tensors of an expert bank (src/experts.rs:146-156); E1 experts each. */
typedef struct {
    const uint32_t *gt, *ut, *dt;           /* [E1][H/16][I/16][32], same, [E1][I/16][H/16][32] */
    const uint16_t *suh_g, *suh_u, *suh_d;  /* [E1][H], [E1][H], [E1][I] */
    const uint16_t *svh_g, *svh_u, *svh_d;  /* [E1][I], [E1][I], [E1][H] */
} gfo_weights;

typedef struct {
    float *wg, *wu, *wd;                    /* unpacked fp32 matrices of one expert */
} expert_mats;

static void expert_unpack(const gfo_weights *W, int e, int H, int I, expert_mats *m, int threads) {
    size_t gsz = (size_t)(H / 16) * (I / 16) * 32;
    m->wg = (float *)malloc((size_t)H * I * sizeof(float));
    m->wu = (float *)malloc((size_t)H * I * sizeof(float));
    m->wd = (float *)malloc((size_t)H * I * sizeof(float));
    unpack_f32(W->gt + (size_t)e * gsz, H, I, m->wg, threads);
    unpack_f32(W->ut + (size_t)e * gsz, H, I, m->wu, threads);
    unpack_f32(W->dt + (size_t)e * gsz, I, H, m->wd, threads);
}
static void expert_free(expert_mats *m) { free(m->wg); free(m->wu); free(m->wd); }

/* One activation row through expert e with unpacked matrices: src/experts.rs:100-135.
 * xrow: the row's values (bf16-exact fp32).  y[H] fp32.  xd_out (optional) [I]: the fp16-rounded
 * down-projection input (the device's Xd). */
static void expert_row(const gfo_weights *W, const expert_mats *m, int e, const float *xrow, int H, int I,
                       float limit, int sk_gu, int sk_dn, int mode, float *y, float *xd_out) {
    float *rot = (float *)malloc((size_t)H * sizeof(float));
    float *g = (float *)malloc((size_t)I * sizeof(float));
    float *u = (float *)malloc((size_t)I * sizeof(float));
    float *act = (float *)malloc((size_t)I * sizeof(float));
    rot_in(xrow, W->suh_g + (size_t)e * H, H, rot);
    gfo_matmul(rot, m->wg, H, I, sk_gu, mode, g);
    gfo_had128(g, I);
    rot_in(xrow, W->suh_u + (size_t)e * H, H, rot);
    gfo_matmul(rot, m->wu, H, I, sk_gu, mode, u);
    gfo_had128(u, I);
    for (int n = 0; n < I; ++n) {
        float gg = gfo_bf(g[n] * HAD_SCALE * gfo_f16_to_f32(W->svh_g[(size_t)e * I + n]));
        float uu = gfo_bf(u[n] * HAD_SCALE * gfo_f16_to_f32(W->svh_u[(size_t)e * I + n]));
        gg = fminf(gg, limit);
        uu = fminf(fmaxf(uu, -limit), limit);
        float a = gfo_bf(gfo_bf(gg / (1.f + expf(-gg))) * uu);
        act[n] = a * gfo_f16_to_f32(W->suh_d[(size_t)e * I + n]);
    }
    gfo_had128(act, I);
    for (int n = 0; n < I; ++n) act[n] = gfo_hf(act[n] * HAD_SCALE);
    if (xd_out) memcpy(xd_out, act, (size_t)I * sizeof(float));
    gfo_matmul(act, m->wd, I, H, sk_dn, mode, y);
    gfo_had128(y, H);
    for (int d = 0; d < H; ++d) y[d] = y[d] * HAD_SCALE * gfo_f16_to_f32(W->svh_d[(size_t)e * H + d]);
    free(rot); free(g); free(u); free(act);
}

/* Every pair p = row*slots+slot of a window: Y[p][H] = expert(picks[p])(x[row]).
 * x: bf16 bits [rows][x_stride].  skip_ge: experts with id >= skip_ge are not computed and their Y rows
 * are left untouched (the reference leaves the shared slot to another kernel: native/exl3.cu:151,229).
 * xd (optional): [P][I] fp32 values of the rounded down-projection inputs.
 * threads: 1 = the faithful single-thread path, >1 = OpenMP over pairs of one expert / experts. */
void gfo_experts_run_rows(const gfo_weights *W, int H, int I, int E1, int slots, const uint16_t *x, int x_stride,
                          const int *picks, int rows, int skip_ge, float limit, int sk_gu, int sk_dn, int mode,
                          int threads, float *Y, float *xd) {
    int P = rows * slots;
    if (threads < 1) threads = 1;
    for (int e = 0; e < E1; ++e) {
        if (e >= skip_ge) break;
        int n = 0;
        for (int p = 0; p < P; ++p) n += picks[p] == e;
        if (!n) continue;
        expert_mats m;
        expert_unpack(W, e, H, I, &m, threads);
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
        for (int p = 0; p < P; ++p) {
            if (picks[p] != e) continue;
            int row = p / slots;
            float *xr = (float *)malloc((size_t)H * sizeof(float));
            for (int k = 0; k < H; ++k) xr[k] = gfo_bf16_to_f32(x[(size_t)row * x_stride + k]);
            expert_row(W, &m, e, xr, H, I, limit, sk_gu, sk_dn, mode, Y + (size_t)p * H,
                       xd ? xd + (size_t)p * I : NULL);
            free(xr);
        }
        expert_free(&m);
    }
}

/* Combine (call site src/moe.rs:171-181): out[r] = sum_{s < slots-1} w[r][s] * Y[r][s] + Y[r][slots-1],
 * fp32, ascending slot order, the shared slot last.  weights[rows][slots] (the last entry unused). */
void gfo_combine(const float *Y, const float *weights, int rows, int slots, int H, float *out) {
    for (int r = 0; r < rows; ++r)
        for (int d = 0; d < H; ++d) {
            float acc = 0.f;
            for (int s = 0; s + 1 < slots; ++s)
                acc += weights[r * slots + s] * Y[((size_t)r * slots + s) * H + d];
            out[(size_t)r * H + d] = acc + Y[((size_t)r * slots + slots - 1) * H + d];
        }
}

/* ---------------------------------------------------------------- grouping */

/* Stable grouping (native/grouping.cu:67-100; expectation built as in src/grouping.rs:143-192):
 * ids[u] = distinct expert ids ascending, *count = their number, members[u][0..] = row*32+slot in
 * ascending row order, tails and unused rows -1.  members has E1 rows of maxm.  Returns 0, or -1 when a
 * pick is out of range or an expert has more than maxm members. */
int gfo_grouping(const int *picks, int rows, int slots, int E1, int maxm, int *ids, int *count, int *members) {
    int *n = (int *)calloc((size_t)E1, sizeof(int));
    int *place = (int *)malloc((size_t)E1 * sizeof(int));
    for (size_t i = 0; i < (size_t)E1 * maxm; ++i) members[i] = -1;
    /* one member per (row, expert): a row that names an expert twice counts once, with its first slot
     * (the reference marks a row bit per expert and then looks up the first matching slot) */
    for (int r = 0; r < rows; ++r)
        for (int s = 0; s < slots; ++s) {
            int e = picks[r * slots + s], dup = 0;
            if (e < 0 || e >= E1) { free(n); free(place); return -1; }
            for (int q = 0; q < s; ++q) dup |= picks[r * slots + q] == e;
            if (!dup) n[e]++;
        }
    int u = 0;
    for (int e = 0; e < E1; ++e) {
        place[e] = -1;
        if (n[e]) { if (n[e] > maxm) { free(n); free(place); return -1; } ids[u] = e; place[e] = u++; }
        n[e] = 0;
    }
    *count = u;
    for (int r = 0; r < rows; ++r)
        for (int s = 0; s < slots; ++s) {
            int e = picks[r * slots + s], dup = 0;
            for (int q = 0; q < s; ++q) dup |= picks[r * slots + q] == e;
            if (!dup) members[(size_t)place[e] * maxm + n[e]++] = r * 32 + s;
        }
    free(n); free(place);
    return 0;
}

/* ---------------------------------------------------------------- router (next to the path) */

/* Router logits (call site src/moe.rs:77-95; the reference's kernels here are precompiled without source, so this is
 * the semantic form: PARITY UNPINNED): logits[r][e] = sum_k x[r][k] * wr[e][k], x and wr bf16 (given as their bit
 * patterns), accumulated in double and rounded to fp32. */
void gfo_router_logits(const uint16_t *x, int x_stride, const uint16_t *wr, int rows, int H, int E, float *logits) {
    for (int r = 0; r < rows; ++r)
        for (int e = 0; e < E; ++e) {
            double acc = 0.0;
            for (int k = 0; k < H; ++k) {
                uint32_t a = (uint32_t)x[(size_t)r * x_stride + k] << 16, b = (uint32_t)wr[(size_t)e * H + k] << 16;
                float fa, fb;
                memcpy(&fa, &a, 4); memcpy(&fb, &b, 4);
                acc += (double)fa * (double)fb;
            }
            logits[(size_t)r * E + e] = (float)acc;
        }
}

/* Top-k of the sigmoid router (the benchmark's definition; the reference's _topk has no source: PARITY UNPINNED):
 * the topk largest logits of a row, ties to the lower expert id, in descending order; weight = sigmoid(logit)
 * divided by the sum of the chosen sigmoids (fp32); the row's last slot names the shared expert (id E), weight 1.
 * picks, weights: [rows][topk + 1]. */
void gfo_topk(const float *logits, int rows, int E, int topk, int *picks, float *weights) {
    for (int r = 0; r < rows; ++r) {
        const float *l = logits + (size_t)r * E;
        int *pk = picks + (size_t)r * (topk + 1);
        float *w = weights + (size_t)r * (topk + 1);
        float sum = 0.f;
        for (int j = 0; j < topk; ++j) {
            int best = -1;
            for (int e = 0; e < E; ++e) {
                int taken = 0;
                for (int q = 0; q < j; ++q) taken |= pk[q] == e;
                if (taken) continue;
                if (best < 0 || l[e] > l[best]) best = e;
            }
            pk[j] = best;
            w[j] = 1.f / (1.f + expf(-l[best]));
            sum += w[j];
        }
        for (int j = 0; j < topk; ++j) w[j] = w[j] / sum;
        pk[topk] = E;
        w[topk] = 1.f;
    }
}

int gfo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
