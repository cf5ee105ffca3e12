/*
 * C restatement of the reference's CPU semantics for the quantized-matmul path. TEST INFRASTRUCTURE ONLY: it is the
 * timed CPU baseline of the benchmark and a second checker beside oracle/qref.py; the library never links it.
 *
 * Follows (paths inside the reference project): Sources/Ingot/Loader/Quant.swift:119-202 (bf16, unpack, dequantise,
 * e2m1, e8m0), Tests/IngotTests/KernelHarness.swift:190-195 (Y = X W^T in float), :720-766 (MoE with given routing,
 * h rounded to half), :185-188 (swiglu_oai), Tests/IngotTests/KernelCaseRouter.swift:57-80 (routing rule).
 * The dequantisation sits inside every call: a call does the same work the GPU operator does (unpack + scale + matmul).
 * Parity: pinned against oracle/qref.py in tests/test_oracle_c.py, which is itself pinned on the reference's vectors.
 *
 * Build: make -C oracle/c   (gcc -O3 -fopenmp -shared)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* Number of OpenMP threads the following calls use (launchers such as torch.distributed.run export OMP_NUM_THREADS=1,
 * which would otherwise turn the timed baseline into a one-core run). Returns the count now in force. */
int qo_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

static inline float bf16_to_f32(uint16_t v) {
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round a float to fp16 and back (round to nearest even), for the h rounding of the MoE kernels */
static inline float round_f16(float f) {
    _Float16 h = (_Float16)f;
    return (float)h;
}

static const float E2M1[16] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

static inline float e8m0_to_f32(uint8_t s) { return s == 255 ? NAN : ldexpf(1.0f, (int)s - 127); }

/* Dequantises one weight row (K inputs) into out. mode 0: affine (bits 4/8, or 6 as one little-endian bit stream with
 * value k in bits 6k.. of the row, Loader/Quant.swift:126-136; group 64 or 32), mode 1: mxfp4. */
static void dequant_row(const uint32_t* w, const void* scales, const uint16_t* biases, int mode, int bits, int group,
                        int K, float* out) {
    if (mode == 1) {
        const uint8_t* s = (const uint8_t*)scales;
        for (int k = 0; k < K; k++) {
            const uint32_t q = (w[k >> 3] >> (4 * (k & 7))) & 15u;
            out[k] = e8m0_to_f32(s[k / 32]) * E2M1[q];
        }
        return;
    }
    const uint16_t* s = (const uint16_t*)scales;
    const int per = 32 / bits;
    const uint32_t mask = (1u << bits) - 1u;
    for (int k = 0; k < K; k++) {
        uint32_t q;
        if (32 % bits != 0) {
            const int bit = bits * k, wi = bit / 32, o = bit % 32;
            uint64_t v = (uint64_t)w[wi] >> o;
            if (o + bits > 32) v |= (uint64_t)w[wi + 1] << (32 - o);
            q = (uint32_t)v & mask;
        } else {
            q = (w[k / per] >> (bits * (k % per))) & mask;
        }
        out[k] = bf16_to_f32(s[k / group]) * (float)q + bf16_to_f32(biases[k / group]);
    }
}

static inline float dotf(const float* a, const float* b, int n) {
    double acc = 0.0;
    float p[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int i = 0;
    for (; i + 8 <= n; i += 8)
        for (int j = 0; j < 8; j++) p[j] += a[i + j] * b[i + j];
    for (; i < n; i++) acc += (double)a[i] * b[i];
    for (int j = 0; j < 8; j++) acc += p[j];
    return (float)acc;
}

/* Y[M, N] = X[M, K] * dequant(W)[N, K]^T. x float [M, K]; y float [M, N]. Returns the number of threads used. */
int qo_qmm(const float* x, const uint32_t* w, const void* scales, const uint16_t* biases, int mode, int bits, int group,
           float* y, int M, int N, int K) {
    const int words = K * bits / 32;
    const int groups = K / group;
    const int sbytes = mode == 1 ? 1 : 2;
    int threads = 1;
#pragma omp parallel
    {
#ifdef _OPENMP
#pragma omp single
        threads = omp_get_num_threads();
#endif
        float* row = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(static)
        for (int n = 0; n < N; n++) {
            dequant_row(w + (size_t)n * words, (const char*)scales + (size_t)n * groups * sbytes,
                        biases ? biases + (size_t)n * groups : NULL, mode, bits, group, K, row);
            for (int m = 0; m < M; m++) y[(size_t)m * N + n] = dotf(x + (size_t)m * K, row, K);
        }
        free(row);
    }
    return threads;
}

static inline float act_glu(int act, float g, float u, float limit) {
    if (act == 2) {
        const float gc = g < limit ? g : limit;
        const float uc = u < -limit ? -limit : (u > limit ? limit : u);
        return (uc + 1.0f) * (gc / (1.0f + expf(-1.702f * gc)));
    }
    return g / (1.0f + expf(-g)) * u;
}

/* Routing rule on given logits [T, ld]: top-k, ties to the lower index, NaN = -inf, softmax over the chosen logits. */
void qo_route(const float* logits, int ld, int T, int E, int topk, const float* logit_bias, float scale,
              const float* per_expert_scale, uint32_t* inds, float* wts) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; t++) {
        float v[1024];
        unsigned char taken[1024];
        for (int e = 0; e < E; e++) {
            float f = logits[(size_t)t * ld + e] + (logit_bias ? logit_bias[e] : 0.f);
            v[e] = isnan(f) ? -INFINITY : f;
            taken[e] = 0;
        }
        float top[64];
        for (int k = 0; k < topk; k++) {
            int best = -1;
            for (int e = 0; e < E; e++)
                if (!taken[e] && (best < 0 || v[e] > v[best])) best = e;
            taken[best] = 1;
            inds[(size_t)t * topk + k] = (uint32_t)best;
            top[k] = v[best];
        }
        float ex[64], sum = 0.f;
        for (int k = 0; k < topk; k++) {
            ex[k] = expf(top[k] - top[0]);
            sum += ex[k];
        }
        for (int k = 0; k < topk; k++) {
            float wv = ex[k] / sum * scale;
            if (per_expert_scale) wv *= per_expert_scale[inds[(size_t)t * topk + k]];
            wts[(size_t)t * topk + k] = wv;
        }
    }
}

/* MoE FFN with the routing given. Expert tensors are stacked [E, ...]; mode/bits/group as in qo_qmm.
 * y[t] = sum_k w[t,k] * (down_e(half(act(gate_e x + bg, up_e x + bu))) + bd). Returns the threads used. */
int qo_moe_ffn(const float* x, int T, int D, int I, int E, int topk, const uint32_t* inds, const float* wts,
               const uint32_t* gate_w, const void* gate_s, const uint16_t* gate_b, const uint32_t* up_w, const void* up_s,
               const uint16_t* up_b, const uint32_t* down_w, const void* down_s, const uint16_t* down_b, int mode,
               int group, int act, float limit, const float* bias_g, const float* bias_u, const float* bias_d, float* y) {
    const int sbytes = mode == 1 ? 1 : 2;
    const size_t gw = (size_t)I * (D / 8), gs = (size_t)I * (D / group);
    const size_t dw = (size_t)D * (I / 8), ds = (size_t)D * (I / group);
    const int P = T * topk;
    memset(y, 0, sizeof(float) * (size_t)T * D);
    int threads = 1;
    /* rows grouped by expert */
    int* order = (int*)malloc(sizeof(int) * (size_t)P);
    int* start = (int*)calloc((size_t)E + 1, sizeof(int));
    for (int i = 0; i < P; i++) start[inds[i] + 1]++;
    for (int e = 0; e < E; e++) start[e + 1] += start[e];
    int* fill = (int*)malloc(sizeof(int) * (size_t)E);
    memcpy(fill, start, sizeof(int) * (size_t)E);
    for (int i = 0; i < P; i++) order[fill[inds[i]]++] = i;
    float* h = (float*)malloc(sizeof(float) * (size_t)P * I);
    float* yd = (float*)malloc(sizeof(float) * (size_t)P * D);
#pragma omp parallel
    {
#ifdef _OPENMP
#pragma omp single
        threads = omp_get_num_threads();
#endif
        float* rg = (float*)malloc(sizeof(float) * (size_t)(D > I ? D : I));
        float* ru = (float*)malloc(sizeof(float) * (size_t)(D > I ? D : I));
        /* gate + up + activation: parallel over (expert, output row) */
#pragma omp for schedule(dynamic, 16) collapse(2)
        for (int e = 0; e < E; e++)
            for (int i = 0; i < I; i++) {
                if (start[e + 1] == start[e]) continue;
                dequant_row(gate_w + e * gw + (size_t)i * (D / 8), (const char*)gate_s + (e * gs + (size_t)i * (D / group)) * sbytes,
                            gate_b ? gate_b + e * gs + (size_t)i * (D / group) : NULL, mode, 4, group, D, rg);
                dequant_row(up_w + e * gw + (size_t)i * (D / 8), (const char*)up_s + (e * gs + (size_t)i * (D / group)) * sbytes,
                            up_b ? up_b + e * gs + (size_t)i * (D / group) : NULL, mode, 4, group, D, ru);
                for (int r = start[e]; r < start[e + 1]; r++) {
                    const float* xr = x + (size_t)(order[r] / topk) * D;
                    float g = dotf(xr, rg, D), u = dotf(xr, ru, D);
                    if (bias_g) { g += bias_g[(size_t)e * I + i]; u += bias_u[(size_t)e * I + i]; }
                    h[(size_t)r * I + i] = round_f16(act_glu(act, g, u, limit));
                }
            }
        /* down: parallel over (expert, output row) */
#pragma omp for schedule(dynamic, 16) collapse(2)
        for (int e = 0; e < E; e++)
            for (int d = 0; d < D; d++) {
                if (start[e + 1] == start[e]) continue;
                dequant_row(down_w + e * dw + (size_t)d * (I / 8), (const char*)down_s + (e * ds + (size_t)d * (I / group)) * sbytes,
                            down_b ? down_b + e * ds + (size_t)d * (I / group) : NULL, mode, 4, group, I, rg);
                for (int r = start[e]; r < start[e + 1]; r++) {
                    float v = dotf(h + (size_t)r * I, rg, I);
                    if (bias_d) v += bias_d[(size_t)e * D + d];
                    yd[(size_t)r * D + d] = v;
                }
            }
        free(rg);
        free(ru);
        /* combine in router rank order */
        int* posn = NULL;
#pragma omp single
        {
            posn = (int*)malloc(sizeof(int) * (size_t)P);
            for (int r = 0; r < P; r++) posn[order[r]] = r;
            for (int t = 0; t < T; t++)
                for (int k = 0; k < topk; k++) {
                    const float wv = wts[(size_t)t * topk + k];
                    const float* src = yd + (size_t)posn[t * topk + k] * D;
                    float* dst = y + (size_t)t * D;
                    for (int d = 0; d < D; d++) dst[d] += wv * src[d];
                }
            free(posn);
        }
    }
    free(order); free(start); free(fill); free(h); free(yd);
    return threads;
}
