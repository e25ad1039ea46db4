/* CPU restatement in plain C of the reference's MoE block, TEST INFRASTRUCTURE
 * ONLY: the checker's second implementation and the timed CPU baseline.  It is
 * never linked into or called by the product library.
 *
 * Follows the structure of mlx/src/nn/moe.rs:55-183 as the reference executes
 * it: router matmul + softmax + descending top-k (moe.rs:67-82), host
 * bucketing token-major/slot-minor (moe.rs:93-104), a loop over experts doing
 * take -> gate/up/down quantized matmuls with silu*up in between
 * (moe.rs:117-131, 26-32; linear.rs:51-63 `x @ dequantize(w)^T`), per-token
 * weighted sum in expert order (moe.rs:147-165), gated shared expert
 * (moe.rs:173-181).  Formats: MLX affine 2/3/4/5/6/8-bit, mxfp8, nvfp4
 * (see oracle/formats.py for the layouts).  fp32 accumulation; parity of this
 * file is pinned against oracle/moe.py by tests/test_oracle_c.py (parity with
 * the reference itself is unpinned: MLX is not in the reference tree).
 *
 * Parallelism: OpenMP over tokens (router, combine) and over experts (the
 * expert loop), which is what a multi-threaded CPU backend would do. */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef struct {
    const uint8_t* w;
    const uint8_t* scales;
    const uint8_t* biases;
    float global_scale;
} ref_q;

static inline float bf16_to_f32(uint16_t b) {
    union { uint32_t u; float f; } v;
    v.u = (uint32_t)b << 16;
    return v.f;
}

static float e4m3_to_f32(uint8_t v) {
    int s = v >> 7, e = (v >> 3) & 15, m = v & 7;
    float r = e == 0 ? ldexpf((float)m, -9) : ldexpf(1.0f + m / 8.0f, e - 7);
    return s ? -r : r;
}

static const float E2M1[16] = {0, 0.5f, 1, 1.5f, 2, 3, 4, 6, -0.0f, -0.5f, -1, -1.5f, -2, -3, -4, -6};

/* Dequantize one packed row of `in` values into out[in]. */
static void dequant_row(const ref_q* q, size_t row, int in, int mode, int bits, int group, float* out) {
    const uint8_t* w = q->w + row * ((size_t)in * bits / 8);
    const int ng = in / group;
    if (mode == 0) {
        const uint16_t* s = (const uint16_t*)q->scales + row * ng;
        const uint16_t* b = (const uint16_t*)q->biases + row * ng;
        const uint32_t mask = (1u << bits) - 1u;
        for (int k = 0; k < in; ++k) {
            size_t bit = (size_t)k * bits;
            uint32_t v = w[bit >> 3];
            if ((bit & 7) + bits > 8) v |= (uint32_t)w[(bit >> 3) + 1] << 8;
            float qv = (float)((v >> (bit & 7)) & mask);
            out[k] = qv * bf16_to_f32(s[k / group]) + bf16_to_f32(b[k / group]);
        }
    } else if (mode == 1) {
        const uint8_t* s = q->scales + row * ng;
        for (int k = 0; k < in; ++k) out[k] = e4m3_to_f32(w[k]) * ldexpf(1.0f, (int)s[k / group] - 127);
    } else {
        const uint8_t* s = q->scales + row * ng;
        for (int k = 0; k < in; ++k) {
            uint8_t nib = (k & 1) ? (w[k >> 1] >> 4) : (w[k >> 1] & 15);
            out[k] = (E2M1[nib] * e4m3_to_f32(s[k / group])) * q->global_scale;
        }
    }
}

static inline float dotf(const float* a, const float* b, int n) {
    float acc = 0.f;
    for (int i = 0; i < n; ++i) acc += a[i] * b[i];
    return acc;
}

/* out[m, n_out] = x[m, in] @ dequant(W[row0 .. row0+n_out, in])^T ; wrow: scratch of `in` floats */
static void qmm_t(const float* x, int m, const ref_q* q, size_t row0, int n_out, int in, int mode, int bits,
                  int group, float* out, float* wrow) {
    for (int n = 0; n < n_out; ++n) {
        dequant_row(q, row0 + n, in, mode, bits, group, wrow);
        for (int r = 0; r < m; ++r) out[(size_t)r * n_out + n] = dotf(x + (size_t)r * in, wrow, in);
    }
}

static inline float siluf(float g) { return g / (1.0f + expf(-g)); }

/* SwiGLU MLP on m rows: d = down(silu(gate(x)) * up(x)) */
static void swiglu(const float* x, int m, int H, int I, const ref_q* gate, size_t gate_row0, const ref_q* up,
                   size_t up_row0, const ref_q* down, size_t down_row0, int mode, int bits, int group, float* d,
                   float* tmp /* m*I*2 + max(H,I) floats */) {
    float* g = tmp;
    float* u = tmp + (size_t)m * I;
    float* wrow = u + (size_t)m * I;
    qmm_t(x, m, gate, gate_row0, I, H, mode, bits, group, g, wrow);
    qmm_t(x, m, up, up_row0, I, H, mode, bits, group, u, wrow);
    for (size_t i = 0; i < (size_t)m * I; ++i) g[i] = siluf(g[i]) * u[i];
    qmm_t(g, m, down, down_row0, H, I, mode, bits, group, d, wrow);
}

/* Router in the reference's dtypes (logits and probabilities rounded to bf16 before the selection,
 * moe.rs:67-74 with a bf16 model) instead of fp32; off by default.  Process-wide. */
static int g_bf16_logits = 0;
void moe_ref_set_bf16_logits(int on) { g_bf16_logits = on != 0; }
static inline float round_bf16(float v) {
    uint32_t u;
    memcpy(&u, &v, 4);
    if ((u & 0x7f800000u) != 0x7f800000u) u += 0x7fffu + ((u >> 16) & 1u);   /* to nearest, ties to even */
    u &= 0xffff0000u;
    memcpy(&v, &u, 4);
    return v;
}

int moe_ref_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* y: fp32 [N,H]; top_idx/top_w: [N,k]; perm: [N*k]; counts: [E].  Returns 0. */
int moe_ref_forward(int N, int H, int E, int k, int I, int Is, int norm, int mode, int bits, int group,
                    const uint16_t* x_bf16, const uint16_t* router_w, const float* logit_bias, ref_q gate_up,
                    ref_q down, ref_q sgate, ref_q sup, ref_q sdown, const uint16_t* sg_w, float* y,
                    int32_t* top_idx, float* top_w, int32_t* perm, int32_t* counts) {
    const int A = N * k;
    float* x = (float*)malloc((size_t)N * H * sizeof(float));
    for (size_t i = 0; i < (size_t)N * H; ++i) x[i] = bf16_to_f32(x_bf16[i]);

    /* 1. router: logits, softmax, descending top-k (lower index first among ties), renormalise */
#pragma omp parallel
    {
        float* p = (float*)malloc((size_t)E * sizeof(float));
        float* wr = (float*)malloc((size_t)H * sizeof(float));
#pragma omp for schedule(static)
        for (int t = 0; t < N; ++t) {
            float mx = -INFINITY;
            for (int e = 0; e < E; ++e) {
                for (int c = 0; c < H; ++c) wr[c] = bf16_to_f32(router_w[(size_t)e * H + c]);
                double acc = 0;
                for (int c = 0; c < H; ++c) acc += (double)x[(size_t)t * H + c] * wr[c];
                p[e] = (float)(acc + (logit_bias ? logit_bias[e] : 0.f));
                if (g_bf16_logits) p[e] = round_bf16(p[e]);
                if (p[e] > mx) mx = p[e];
            }
            double sum = 0;
            for (int e = 0; e < E; ++e) sum += exp((double)(p[e] - mx));
            for (int e = 0; e < E; ++e) {
                p[e] = (float)(exp((double)(p[e] - mx)) / sum);
                if (g_bf16_logits) p[e] = round_bf16(p[e]);
            }
            double wsum = 0;
            for (int s = 0; s < k; ++s) {
                int best = -1;
                for (int e = 0; e < E; ++e)
                    if (p[e] >= 0.f && (best < 0 || p[e] > p[best])) best = e;
                top_idx[(size_t)t * k + s] = best;
                top_w[(size_t)t * k + s] = p[best];
                wsum += p[best];
                p[best] = -1.f;
            }
            if (norm)
                for (int s = 0; s < k; ++s) top_w[(size_t)t * k + s] = (float)(top_w[(size_t)t * k + s] / wsum);
        }
        free(p);
        free(wr);
    }

    /* 2. bucketing: stable counting sort of flat assignment indices by expert */
    int32_t* offsets = (int32_t*)calloc((size_t)E + 1, sizeof(int32_t));
    memset(counts, 0, (size_t)E * sizeof(int32_t));
    for (int f = 0; f < A; ++f) counts[top_idx[f]]++;
    for (int e = 0; e < E; ++e) offsets[e + 1] = offsets[e] + counts[e];
    int32_t* fill = (int32_t*)malloc((size_t)E * sizeof(int32_t));
    memcpy(fill, offsets, (size_t)E * sizeof(int32_t));
    for (int f = 0; f < A; ++f) perm[fill[top_idx[f]]++] = f;
    free(fill);

    /* 3. expert loop */
    float* rows = (float*)malloc((size_t)A * H * sizeof(float));
    const int mid_max = I > Is ? I : Is;
#pragma omp parallel for schedule(dynamic, 1)
    for (int e = 0; e < E; ++e) {
        const int lo = offsets[e], m = offsets[e + 1] - lo;
        if (m == 0) continue;
        float* xe = (float*)malloc((size_t)m * H * sizeof(float));
        float* tmp = (float*)malloc(((size_t)m * I * 2 + (H > mid_max ? H : mid_max)) * sizeof(float));
        for (int r = 0; r < m; ++r) memcpy(xe + (size_t)r * H, x + (size_t)(perm[lo + r] / k) * H, (size_t)H * sizeof(float));
        swiglu(xe, m, H, I, &gate_up, (size_t)e * 2 * I, &gate_up, (size_t)e * 2 * I + I, &down, (size_t)e * H, mode,
               bits, group, rows + (size_t)lo * H, tmp);
        free(xe);
        free(tmp);
    }

    /* 4. shared expert on all tokens (token blocks in parallel) */
    float* shared = NULL;
    if (Is > 0) {
        shared = (float*)malloc((size_t)N * H * sizeof(float));
        const int blk = 8;
#pragma omp parallel for schedule(dynamic, 1)
        for (int t0 = 0; t0 < N; t0 += blk) {
            const int m = N - t0 < blk ? N - t0 : blk;
            float* tmp = (float*)malloc(((size_t)m * Is * 2 + (H > mid_max ? H : mid_max)) * sizeof(float));
            swiglu(x + (size_t)t0 * H, m, H, Is, &sgate, 0, &sup, 0, &sdown, 0, mode, bits, group, shared + (size_t)t0 * H,
                   tmp);
            free(tmp);
        }
    }

    /* 5. combine: per token, rows in ascending sorted-slot (= expert) order, then the gated shared row */
    int32_t* inv = (int32_t*)malloc((size_t)A * sizeof(int32_t));
    for (int j = 0; j < A; ++j) inv[perm[j]] = j;
#pragma omp parallel for schedule(static)
    for (int t = 0; t < N; ++t) {
        int slots[64];
        for (int s = 0; s < k; ++s) {
            int v = inv[(size_t)t * k + s], j = s;
            while (j > 0 && slots[j - 1] > v) { slots[j] = slots[j - 1]; --j; }
            slots[j] = v;
        }
        float gate = 0.f;
        if (Is > 0) {
            double acc = 0;
            for (int c = 0; c < H; ++c) acc += (double)x[(size_t)t * H + c] * bf16_to_f32(sg_w[c]);
            gate = (float)(1.0 / (1.0 + exp(-acc)));
        }
        for (int c = 0; c < H; ++c) {
            float acc = 0.f;
            for (int s = 0; s < k; ++s) acc += rows[(size_t)slots[s] * H + c] * top_w[perm[slots[s]]];
            if (Is > 0) acc += shared[(size_t)t * H + c] * gate;
            y[(size_t)t * H + c] = acc;
        }
    }
    free(inv);
    free(shared);
    free(rows);
    free(offsets);
    free(x);
    return 0;
}
