/* linear_oracle.c — CPU restatement of vAi's Linear arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is
 * compared against and the timed CPU baseline; nothing in the shipped library
 * links, imports or calls it.
 *
 * The reference has no CPU implementation of this path: its arithmetic lives
 * in GLSL compute shaders.  Each function below restates one of them in plain
 * C and cites the lines it follows (paths inside the vAi source tree).
 *
 * Pinning: the reference commits no golden vectors for Linear.  Its own tests
 * pin the node against float64 torch.nn.functional.linear + epilogue
 * (python/tests/node_check.py:128-131, python/tests/nodes/test_linear.py:34-35).
 * The fixtures in tests/golden/ are produced by importing those reference test
 * files and running their draw order and reference functions; this oracle is
 * checked against them.
 *
 * Build: gcc -O3 -march=native -fopenmp -shared -fPIC (see oracle/build_oracle.py).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* dtype codes: vai/engine/tensor.h:19 (Fp32=0, Fp16=1, None=2); bf16 appended. */
enum { DT_F32 = 0, DT_F16 = 1, DT_NONE = 2, DT_BF16 = 3 };

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float    u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* fp32 -> fp16: round to nearest even, subnormal results flush to zero,
 * overflow saturates to inf, NaN/Inf kept (vai/engine/tensor.cpp:46-69). */
uint16_t vai_oracle_f32_to_f16(float f)
{
    const uint32_t b = f2u(f);
    const uint32_t sign = (b >> 16) & 0x8000u;
    const uint32_t exp_raw = (b >> 23) & 0xFFu;
    const uint32_t mant = b & 0x7FFFFFu;
    if (exp_raw == 0xFFu) return (uint16_t)(sign | 0x7C00u | (mant ? 0x0200u : 0u));
    const int32_t e = (int32_t)exp_raw - 112;
    if (e <= 0) return (uint16_t)sign;
    const uint32_t rest = mant & 0x1FFFu;
    uint32_t m10 = mant >> 13;
    if (rest > 0x1000u || (rest == 0x1000u && (m10 & 1u))) m10++;
    uint32_t out = (uint32_t)e * 0x400u + m10;
    if (out >= 0x7C00u) out = 0x7C00u;
    return (uint16_t)(sign | out);
}

/* fp16 -> fp32, exact (IEEE binary16, subnormals included). */
float vai_oracle_f16_to_f32(uint16_t h)
{
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1Fu;
    uint32_t m = h & 0x3FFu;
    if (e == 0) {
        if (m == 0) return u2f(sign);
        int shift = 0;
        while (!(m & 0x400u)) { m <<= 1; shift++; }
        m &= 0x3FFu;
        return u2f(sign | ((uint32_t)(113 - shift) << 23) | (m << 13));
    }
    if (e == 31) return u2f(sign | 0x7F800000u | (m << 13));
    return u2f(sign | ((e + 112u) << 23) | (m << 13));
}

/* fp32 -> bf16 round to nearest even, NaN quieted (vai/engine/tensor.cpp:73-85). */
uint16_t vai_oracle_f32_to_bf16(float f)
{
    uint32_t b = f2u(f);
    if (((b >> 23) & 0xFFu) == 0xFFu && (b & 0x7FFFFFu)) return (uint16_t)((b >> 16) | 0x40u);
    return (uint16_t)((b + 0x7FFFu + ((b >> 16) & 1u)) >> 16);
}
float vai_oracle_bf16_to_f32(uint16_t b) { return u2f((uint32_t)b << 16); }

void vai_oracle_convert_f32(const float* src, void* dst, int dtype, size_t n)
{
    if (dtype == DT_F32) { memcpy(dst, src, n * 4); return; }
    uint16_t* d = (uint16_t*)dst;
    if (dtype == DT_F16) for (size_t i = 0; i < n; ++i) d[i] = vai_oracle_f32_to_f16(src[i]);
    else                 for (size_t i = 0; i < n; ++i) d[i] = vai_oracle_f32_to_bf16(src[i]);
}

void vai_oracle_widen_f32(const void* src, int dtype, float* dst, size_t n)
{
    if (dtype == DT_F32) { memcpy(dst, src, n * 4); return; }
    const uint16_t* s = (const uint16_t*)src;
    if (dtype == DT_F16) for (size_t i = 0; i < n; ++i) dst[i] = vai_oracle_f16_to_f32(s[i]);
    else                 for (size_t i = 0; i < n; ++i) dst[i] = vai_oracle_bf16_to_f32(s[i]);
}

static inline float load_elem(const void* p, int dtype, size_t i)
{
    if (dtype == DT_F32) return ((const float*)p)[i];
    if (dtype == DT_F16) return vai_oracle_f16_to_f32(((const uint16_t*)p)[i]);
    return vai_oracle_bf16_to_f32(((const uint16_t*)p)[i]);
}
static inline void store_elem(void* p, int dtype, size_t i, float v)
{
    if (dtype == DT_F32) ((float*)p)[i] = v;
    else if (dtype == DT_F16) ((uint16_t*)p)[i] = vai_oracle_f32_to_f16(v);
    else ((uint16_t*)p)[i] = vai_oracle_f32_to_bf16(v);
}
/* value after a round trip through the output dtype (partials are stored in
 * oDtype: vai/nodes/linear.h:2697-2698, linear-reduce.comp:62). */
static inline float round_to(int dtype, float v)
{
    if (dtype == DT_F32) return v;
    if (dtype == DT_F16) return vai_oracle_f16_to_f32(vai_oracle_f32_to_f16(v));
    return vai_oracle_bf16_to_f32(vai_oracle_f32_to_bf16(v));
}

/* Epilogue functions, fp32 (vai/shaders/common/activation.h:19-58). */
static inline float erf_approx(float x)   /* Abramowitz-Stegun 7.1.26, activation.h:19-24 */
{
    const float t = 1.0f / (1.0f + 0.3275911f * fabsf(x));
    const float p = ((((1.061405429f * t - 1.453152027f) * t + 1.421413741f) * t - 0.284496736f) * t + 0.254829592f) * t;
    const float s = (x > 0.0f) ? 1.0f : ((x < 0.0f) ? -1.0f : 0.0f);
    return s * (1.0f - p * expf(-x * x));
}
float vai_oracle_epilogue(int code, float x)   /* activation.h:48-58 */
{
    switch (code) {
    case 1: return x > 0.0f ? x : 0.0f;
    case 2: return 0.5f * x * (1.0f + erf_approx(x * 0.707106781186547524400844f));
    case 3: { const float c = 0.797884560802865355879892f;
              return 0.5f * x * (1.0f + tanhf(c * (x + 0.044715f * x * x * x))); }
    case 4: return x / (1.0f + expf(-x));
    case 5: return 1.0f / (1.0f + expf(-x));
    default: return x;
    }
}

typedef struct {
    uint32_t M, N, K;
    int32_t  i_dtype, w_dtype, o_dtype, b_dtype;
    int32_t  has_bias;
    uint32_t bias_elems;       /* 0: covers O (linear.h:2333-2338) */
    int32_t  has_residual;
    uint32_t residual_elems;
    int32_t  residual_order;   /* 0 after, 1 before the epilogue */
    int32_t  epilogue;
    float    scalar_scale;
    uint32_t split_size;
    int32_t  gate_fuse;
} oracle_desc;

static inline float finish(const oracle_desc* d, float acc, float r)
{
    /* linear-slab.comp:239-241 == linear-reduce.comp:111-112 */
    return d->residual_order == 1 ? d->scalar_scale * vai_oracle_epilogue(d->epilogue, acc + r)
                                  : d->scalar_scale * vai_oracle_epilogue(d->epilogue, acc) + r;
}
static inline float read_bias(const oracle_desc* d, const void* bias, size_t idx)
{
    if (!d->has_bias) return 0.0f;
    return load_elem(bias, d->b_dtype, d->bias_elems ? idx % d->bias_elems : idx);
}
static inline float read_res(const oracle_desc* d, const void* res, size_t idx)
{
    if (!d->has_residual) return 0.0f;
    return load_elem(res, d->o_dtype, d->residual_elems ? idx % d->residual_elems : idx);
}

/* Slab kernel (M <= 8), vai/shaders/linear-slab.comp:118-243.
 * wg_size threads split K in 4-wide chunks strided by the workgroup
 * (linear-slab.comp:118-137, 167-201); each keeps an fp32 partial; subgroupAdd
 * over 32 lanes, then thread 0 folds the per-subgroup sums in order
 * (203-229); thread 0 adds bias, applies epilogue / residual / scale (231-243).
 * subgroupAdd's internal order is unspecified by Vulkan: a pairwise butterfly
 * is used here. */
int vai_oracle_linear_slab(const oracle_desc* d, const void* I, const void* W, const void* bias,
                           const void* R, void* O, uint32_t wg_size)
{
    if (d->M == 0 || d->M > 8 || wg_size == 0 || wg_size % 32u || wg_size > 1024u) return 1;
    const uint32_t M = d->M, N = d->N, K = d->K;
    float* Iw = (float*)malloc((size_t)M * K * sizeof(float));
    if (!Iw) return 2;
    vai_oracle_widen_f32(I, d->i_dtype, Iw, (size_t)M * K);
    const uint32_t chunks = (K + 3u) / 4u;
#pragma omp parallel
    {
        float* lane = (float*)malloc(sizeof(float) * wg_size);
        float* wrow = (float*)malloc(sizeof(float) * K);
#pragma omp for schedule(static)
        for (uint32_t n = 0; n < N; ++n) {
            vai_oracle_widen_f32((const char*)W + (size_t)n * K * (d->w_dtype == DT_F32 ? 4 : 2), d->w_dtype, wrow, K);
            for (uint32_t j = 0; j < M; ++j) {
                const float* x = Iw + (size_t)j * K;
                for (uint32_t t = 0; t < wg_size; ++t) lane[t] = 0.0f;
                /* thread t takes chunks t, t + wg, t + 2 wg, ...: sweeping the chunks in
                 * order visits the lanes round-robin, each lane's sum in its own order */
                const uint32_t full = K / 4u;            /* chunks with no masked element */
                uint32_t c = 0;
                for (; c + wg_size <= full; c += wg_size) {
                    const float* wp = wrow + (size_t)c * 4u;
                    const float* xp = x + (size_t)c * 4u;
#pragma omp simd
                    for (uint32_t t = 0; t < wg_size; ++t) {
                        /* dot(vec4, vec4) left to right */
                        const float dot = ((wp[4 * t] * xp[4 * t] + wp[4 * t + 1] * xp[4 * t + 1]) + wp[4 * t + 2] * xp[4 * t + 2]) +
                                          wp[4 * t + 3] * xp[4 * t + 3];
                        lane[t] += dot;
                    }
                }
                for (; c < chunks; ++c) {
                    const uint32_t t = c % wg_size, k0 = c * 4u;
                    float dot = 0.0f;                    /* K tail masked to 0 (linear-slab.comp:98-116) */
                    for (uint32_t e = 0; e < 4u; ++e)
                        if (k0 + e < K) dot += wrow[k0 + e] * x[k0 + e];
                    lane[t] += dot;
                }
                float acc = 0.0f;
                for (uint32_t sg = 0; sg < wg_size / 32u; ++sg) {
                    float v[32];
                    for (int l = 0; l < 32; ++l) v[l] = lane[sg * 32u + l];
                    for (int off = 16; off > 0; off >>= 1)
                        for (int l = 0; l < off; ++l) v[l] += v[l + off];
                    acc += v[0];
                }
                const size_t idx = (size_t)j * N + n;
                store_elem(O, d->o_dtype, idx, finish(d, acc + read_bias(d, bias, idx), read_res(d, R, idx)));
            }
        }
        free(lane); free(wrow);
    }
    free(Iw);
    return 0;
}

/* Tile kernel + reduce pass (M > 8).
 * GEMM: P[z] = I . W^T over K span z, fp32 accumulate, k ascending
 * (vai/shaders/linear-tile.comp:289-295).  stage_f16 != 0 restates the
 * cooperative-matrix kernel's staging, where both operands are rounded to the
 * 16-bit staging type before the multiply (vai/shaders/linear-cm-nv.comp:128-140);
 * stage_dtype picks fp16 (reference) or bf16 (extension).
 * Reduce: start from bias, add partials in z order, epilogue / residual / scale
 * (vai/shaders/linear-reduce.comp:88-116).  Partials are stored in oDtype when a
 * reduce pass runs (linear.h:2674-2698); with no split and a plain output the
 * GEMM writes O directly (linear.h:300-316). */
int vai_oracle_linear_tile(const oracle_desc* d, const void* I, const void* W, const void* bias,
                           const void* R, void* O, int stage_16, int stage_dtype)
{
    const uint32_t M = d->M, N = d->N, K = d->K;
    if (M == 0 || N == 0 || K == 0) return 1;
    uint32_t split = d->split_size ? d->split_size : K;
    if (split > K) split = K;
    const uint32_t nsplit = (K + split - 1u) / split;
    const int plain = !d->has_bias && !d->has_residual && d->epilogue == 0 && d->scalar_scale == 1.0f;
    const int reduce = nsplit > 1u || !plain;
    float* Iw = (float*)malloc((size_t)M * K * sizeof(float));
    if (!Iw) return 2;
    vai_oracle_widen_f32(I, d->i_dtype, Iw, (size_t)M * K);
    if (stage_16)
        for (size_t i = 0; i < (size_t)M * K; ++i) Iw[i] = round_to(stage_dtype, Iw[i]);
#pragma omp parallel
    {
        float* wrow = (float*)malloc(sizeof(float) * K);
#pragma omp for schedule(static)
        for (uint32_t n = 0; n < N; ++n) {
            vai_oracle_widen_f32((const char*)W + (size_t)n * K * (d->w_dtype == DT_F32 ? 4 : 2), d->w_dtype, wrow, K);
            if (stage_16) for (uint32_t k = 0; k < K; ++k) wrow[k] = round_to(stage_dtype, wrow[k]);
            for (uint32_t m = 0; m < M; ++m) {
                const float* x = Iw + (size_t)m * K;
                const size_t idx = (size_t)m * N + n;
                float total = reduce ? read_bias(d, bias, idx) : 0.0f;
                for (uint32_t z = 0; z < nsplit; ++z) {
                    const uint32_t k1 = (z + 1u) * split < K ? (z + 1u) * split : K;
                    float p = 0.0f;
                    for (uint32_t k = z * split; k < k1; ++k) p += x[k] * wrow[k];
                    total += reduce ? round_to(d->o_dtype, p) : p;
                }
                store_elem(O, d->o_dtype, idx, reduce ? finish(d, total, read_res(d, R, idx)) : total);
            }
        }
        free(wrow);
    }
    free(Iw);
    return 0;
}

/* Linear followed by GatedMul: T = Linear(I) of width 2H, then
 * O[r, j] = epilogue(T[r, j]) * T[r, H + j] (vai/nodes/gated-mul.h:9-20,
 * vai/shaders/gated-mul.comp:1-49).  The Linear itself runs plain
 * (gateValue has no epilogue: vai/groups/gated-feed-forward.h:38); T is kept in
 * `t_dtype`, the dtype the intermediate tensor would have.  With t_dtype = fp32
 * this is the arithmetic the fused CUDA epilogue performs. */
int vai_oracle_linear_gated(const oracle_desc* d, const void* I, const void* W, const void* bias,
                            void* O, int t_dtype, int stage_16, int stage_dtype)
{
    if (d->N % 2u) return 1;
    const uint32_t H = d->N / 2u;
    oracle_desc lin = *d;
    lin.o_dtype = t_dtype; lin.epilogue = 0; lin.has_residual = 0; lin.scalar_scale = 1.0f; lin.gate_fuse = 0;
    void* T = malloc((size_t)d->M * d->N * 4u);
    if (!T) return 2;
    int rc = d->M <= 8 ? vai_oracle_linear_slab(&lin, I, W, bias, NULL, T, 128)
                       : vai_oracle_linear_tile(&lin, I, W, bias, NULL, T, stage_16, stage_dtype);
    if (rc == 0)
        for (uint32_t r = 0; r < d->M; ++r)
            for (uint32_t j = 0; j < H; ++j) {
                const float g = load_elem(T, t_dtype, (size_t)r * d->N + j);
                const float u = load_elem(T, t_dtype, (size_t)r * d->N + H + j);
                store_elem(O, d->o_dtype, (size_t)r * H + j, d->scalar_scale * (vai_oracle_epilogue(d->epilogue, g) * u));
            }
    free(T);
    return rc;
}

/* Path choice of Linear::prepare() on NVIDIA: M <= 8 -> slab, else tile
 * (vai/nodes/linear.h:320, 2355, 2395).  Slab workgroup: 4 subgroups when
 * N <= 8192 && K >= 1024, else 1 (linear.h:655-663).  fp32 x fp32 stages fp32
 * (linear.h:2430-2432); any 16-bit operand stages 16-bit. */
int vai_oracle_linear(const oracle_desc* d, const void* I, const void* W, const void* bias,
                      const void* R, void* O)
{
    if (d->gate_fuse) return vai_oracle_linear_gated(d, I, W, bias, O, DT_F32,
                                                     !(d->i_dtype == DT_F32 && d->w_dtype == DT_F32) && d->M > 8,
                                                     d->w_dtype == DT_F32 ? d->i_dtype : d->w_dtype);
    if (d->M <= 8) {
        const uint32_t wg = (d->N <= 8192u && d->K >= 1024u) ? 128u : 32u;
        return vai_oracle_linear_slab(d, I, W, bias, R, O, wg);
    }
    const int stage16 = !(d->i_dtype == DT_F32 && d->w_dtype == DT_F32);
    return vai_oracle_linear_tile(d, I, W, bias, R, O, stage16, d->w_dtype == DT_F32 ? d->i_dtype : d->w_dtype);
}

/* Argmax node (vai/shaders/argmax.comp:50-95): 256 threads each scan a strided slice of
 * the row keeping the first strict maximum, then a tree merge keeps the lower thread's
 * candidate unless the other is strictly greater.  With ties between different threads
 * the shader's result therefore depends on thread order, not on index order; distinct
 * values (the case the reference tests) give the plain argmax. */
int vai_oracle_argmax(const void* in, int dtype, uint32_t M, uint32_t N, uint32_t* out)
{
    enum { LOCAL = 256 };
    for (uint32_t row = 0; row < M; ++row) {
        float smax[LOCAL];
        uint32_t sidx[LOCAL];
        for (uint32_t tid = 0; tid < LOCAL; ++tid) {
            float best = -3.4028235e38f;
            uint32_t bi = 0;
            for (uint32_t i = tid; i < N; i += LOCAL) {
                const float v = load_elem(in, dtype, (size_t)row * N + i);
                if (v > best) { best = v; bi = i; }
            }
            smax[tid] = best; sidx[tid] = bi;
        }
        for (uint32_t stride = LOCAL / 2; stride > 0; stride >>= 1)
            for (uint32_t tid = 0; tid < stride; ++tid)
                if (smax[tid + stride] > smax[tid]) { smax[tid] = smax[tid + stride]; sidx[tid] = sidx[tid + stride]; }
        out[row] = sidx[0];
    }
    return 0;
}

/* RmsNorm (vai/shaders/rms-norm.comp:92-175): wg_size threads accumulate strided partial
 * sums of squares in fp32, subgroupAdd over 32 lanes (pairwise here), the per-subgroup
 * sums are added in order, invRms = inversesqrt(sum / F + eps), then
 * O = I * invRms * scale + shift + R, evaluated left to right in fp32. */
int vai_oracle_rms_norm(const void* in, const void* scale, const void* shift, const void* res, void* out,
                        uint32_t rows, uint32_t feat, int i_dtype, int w_dtype, int o_dtype, float eps, uint32_t wg_size)
{
    if (wg_size == 0 || wg_size % 32u || wg_size > 1024u) return 1;
    float* lane = (float*)malloc(sizeof(float) * wg_size);
    if (!lane) return 2;
    for (uint32_t row = 0; row < rows; ++row) {
        const size_t base = (size_t)row * feat;
        for (uint32_t t = 0; t < wg_size; ++t) lane[t] = 0.0f;
        for (uint32_t j = 0; j < feat; ++j) {
            const float x = load_elem(in, i_dtype, base + j);
            lane[j % wg_size] += x * x;
        }
        float q = 0.0f;
        for (uint32_t sg = 0; sg < wg_size / 32u; ++sg) {
            float v[32];
            for (int l = 0; l < 32; ++l) v[l] = lane[sg * 32u + l];
            for (int off = 16; off > 0; off >>= 1)
                for (int l = 0; l < off; ++l) v[l] += v[l + off];
            q += v[0];
        }
        const float inv = 1.0f / sqrtf(q / (float)feat + eps);
        for (uint32_t j = 0; j < feat; ++j) {
            float v = load_elem(in, i_dtype, base + j) * inv;
            v = v * (scale ? load_elem(scale, w_dtype, j) : 1.0f);
            v = v + (shift ? load_elem(shift, w_dtype, j) : 0.0f);
            v = v + (res ? load_elem(res, i_dtype, base + j) : 0.0f);
            store_elem(out, o_dtype, base + j, v);
        }
    }
    free(lane);
    return 0;
}

/* LayerNorm (vai/shaders/layer-norm.comp:138-196): shifted one-pass statistics with
 * s = I[row, 0]: wg_size threads accumulate strided partials of sum = S(x - s) and
 * sumSq = S(x - s)^2 in fp32, subgroupAdd over 32 lanes (pairwise here), per-subgroup
 * sums added in order; mean = s + sum / F, m2 = max(sumSq - sum^2 / F, 0),
 * invStd = inversesqrt(m2 / F + eps); then
 * O = (I - mean) * invStd * scale + shift + R left to right in fp32 (layer-norm.comp:132-135).
 * wg_size follows lnTuning (vai/nodes/layer-norm.h:73-88): the power of two >= F / 4
 * within [32, 512]; the caller passes it. */
int vai_oracle_layer_norm(const void* in, const void* scale, const void* shift, const void* res, void* out,
                          uint32_t rows, uint32_t feat, int i_dtype, int w_dtype, int o_dtype, float eps, uint32_t wg_size)
{
    if (wg_size == 0 || wg_size % 32u || wg_size > 1024u || !scale) return 1;
    float* lane = (float*)malloc(sizeof(float) * wg_size * 2u);
    if (!lane) return 2;
    float* lane_sq = lane + wg_size;
    for (uint32_t row = 0; row < rows; ++row) {
        const size_t base = (size_t)row * feat;
        const float sh = load_elem(in, i_dtype, base);
        for (uint32_t t = 0; t < wg_size; ++t) { lane[t] = 0.0f; lane_sq[t] = 0.0f; }
        for (uint32_t j = 0; j < feat; ++j) {
            const float d = load_elem(in, i_dtype, base + j) - sh;
            lane[j % wg_size] += d;
            lane_sq[j % wg_size] += d * d;
        }
        float s = 0.0f, q = 0.0f;
        for (uint32_t sg = 0; sg < wg_size / 32u; ++sg) {
            float v[32], w[32];
            for (int l = 0; l < 32; ++l) { v[l] = lane[sg * 32u + l]; w[l] = lane_sq[sg * 32u + l]; }
            for (int off = 16; off > 0; off >>= 1)
                for (int l = 0; l < off; ++l) { v[l] += v[l + off]; w[l] += w[l + off]; }
            s += v[0];
            q += w[0];
        }
        float m2 = q - s * s / (float)feat;
        if (m2 < 0.0f) m2 = 0.0f;
        const float mean = sh + s / (float)feat;
        const float inv = 1.0f / sqrtf(m2 / (float)feat + eps);
        for (uint32_t j = 0; j < feat; ++j) {
            float v = (load_elem(in, i_dtype, base + j) - mean) * inv * load_elem(scale, w_dtype, j);
            v = v + (shift ? load_elem(shift, w_dtype, j) : 0.0f);
            v = v + (res ? load_elem(res, i_dtype, base + j) : 0.0f);
            store_elem(out, o_dtype, base + j, v);
        }
    }
    free(lane);
    return 0;
}

/* TopKSampling — parity unpinned: the reference holds no test, fixture or golden vector for this
 * node, so this restatement is checked only against a float64 formulation of the same rules.
 * (vai/shaders/topk-sampling.comp:76-79, 237-258): the k best of each row in
 * strict (value descending, index ascending) order, found here by k selection sweeps; then
 * invT = 1 / max(temperature, 1e-6), Z = sum exp((v_r - v_0) * invT) in rank order, and the
 * first rank whose running sum reaches u * Z (rank 0 if none does).  fp32 throughout, expf
 * as the shader's exp.  `in` is fp32 (the caller widens 16-bit logits). */
int vai_oracle_topk_sample(const float* in, uint32_t M, uint32_t N, uint32_t K, float temperature, float u, uint32_t* out)
{
    const uint32_t k = K < N ? K : N;
    if (k == 0 || k > 128u) return 1;
    float top_v[128];
    uint32_t top_i[128];
    for (uint32_t row = 0; row < M; ++row) {
        const float* x = in + (size_t)row * N;
        for (uint32_t r = 0; r < k; ++r) {
            float bv = -3.4028235e38f;
            uint32_t bi = 0xFFFFFFFFu;
            for (uint32_t i = 0; i < N; ++i) {
                const float v = x[i];
                /* ranked strictly below the previous winner ... */
                if (r > 0 && !(v < top_v[r - 1] || (v == top_v[r - 1] && i > top_i[r - 1]))) continue;
                /* ... and the best of those */
                if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
            }
            top_v[r] = bv;
            top_i[r] = bi;
        }
        const float inv_t = 1.0f / (temperature > 1e-6f ? temperature : 1e-6f);
        const float m = top_v[0];
        float z = 0.0f;
        for (uint32_t r = 0; r < k; ++r) z += expf((top_v[r] - m) * inv_t);
        const float target = u * z;
        float cum = 0.0f;
        uint32_t chosen = top_i[0];
        for (uint32_t r = 0; r < k; ++r) {
            cum += expf((top_v[r] - m) * inv_t);
            if (cum >= target) { chosen = top_i[r]; break; }
        }
        out[row] = chosen;
    }
    return 0;
}

/* TopKSampling over a vocabulary split across GPUs (no counterpart in the single-device reference;
 * the same rules applied in two steps).  Step 1, per slab: the k best of each row of the slab's
 * logits [M, n_slab] in (value descending, index ascending) order with index_base added to the
 * column index; a slab narrower than k pads its list with (lowest float, 0xFFFFFFFF).  Step 2:
 * merge `groups` such lists per row (list g of row m at vals / idxs [g * group_stride + m * k]) into the k
 * best of their union in the same order, then the reference's softmax + inverse-CDF sample
 * (vai/shaders/topk-sampling.comp:237-258).  The top-k of a union lies within the union of the
 * parts' top-k, so the two steps give exactly what vai_oracle_topk_sample gives on whole rows. */
int vai_oracle_topk_candidates(const float* in, uint32_t M, uint32_t N, uint32_t K, uint32_t index_base, float* out_val,
                               uint32_t* out_idx)
{
    if (K == 0 || K > 128u) return 1;
    for (uint32_t row = 0; row < M; ++row) {
        const float* x = in + (size_t)row * N;
        float* tv = out_val + (size_t)row * K;
        uint32_t* ti = out_idx + (size_t)row * K;
        for (uint32_t r = 0; r < K; ++r) {
            float bv = -3.4028235e38f;
            uint32_t bi = 0xFFFFFFFFu;
            if (r < N)
                for (uint32_t i = 0; i < N; ++i) {
                    const float v = x[i];
                    const uint32_t gi = index_base + i;
                    if (r > 0 && !(v < tv[r - 1] || (v == tv[r - 1] && gi > ti[r - 1]))) continue;
                    if (v > bv || (v == bv && gi < bi)) { bv = v; bi = gi; }
                }
            tv[r] = bv;
            ti[r] = bi;
        }
    }
    return 0;
}

int vai_oracle_topk_merge_sample(const float* vals, const uint32_t* idxs, uint32_t groups, size_t group_stride, uint32_t M,
                                 uint32_t list_len, uint32_t K, float temperature, float u, uint32_t* out)
{
    if (K == 0 || K > 128u || groups == 0 || list_len == 0) return 1;
    float top_v[128];
    uint32_t top_i[128];
    uint32_t pos[64];
    if (groups > 64u) return 1;
    for (uint32_t row = 0; row < M; ++row) {
        for (uint32_t g = 0; g < groups; ++g) pos[g] = 0;
        for (uint32_t r = 0; r < K; ++r) {
            float bv = -3.4028235e38f;
            uint32_t bi = 0xFFFFFFFFu, bg = 0xFFFFFFFFu;
            for (uint32_t g = 0; g < groups; ++g) {
                if (pos[g] >= list_len) continue;
                const size_t at = (size_t)g * group_stride + (size_t)row * list_len + pos[g];
                const float v = vals[at];
                const uint32_t i = idxs[at];
                if (i == 0xFFFFFFFFu) continue;                       /* padding of a narrow slab */
                if (bg == 0xFFFFFFFFu || v > bv || (v == bv && i < bi)) { bv = v; bi = i; bg = g; }
            }
            top_v[r] = bv;
            top_i[r] = bi;
            if (bg != 0xFFFFFFFFu) pos[bg]++;
        }
        const float inv_t = 1.0f / (temperature > 1e-6f ? temperature : 1e-6f);
        const float m = top_v[0];
        float z = 0.0f;
        for (uint32_t r = 0; r < K; ++r) z += expf((top_v[r] - m) * inv_t);
        const float target = u * z;
        float cum = 0.0f;
        uint32_t chosen = top_i[0];
        for (uint32_t r = 0; r < K; ++r) {
            cum += expf((top_v[r] - m) * inv_t);
            if (cum >= target) { chosen = top_i[r]; break; }
        }
        out[row] = chosen;
    }
    return 0;
}

/* GatedMul as a node of its own (vai/shaders/gated-mul.comp:38-49): one output element
 * per thread, row = e / H, src = row * 2H + (e - row * H); O[e] = epilogue(I[src]) * I[src + H]
 * in fp32, I and O in their own dtypes. */
int vai_oracle_gated_mul(const void* in, void* out, uint32_t rows, uint32_t H, int i_dtype, int o_dtype, int epilogue)
{
    if (!in || !out || rows == 0 || H == 0) return 1;
    const size_t total = (size_t)rows * H;
    for (size_t e = 0; e < total; ++e) {
        const size_t row = e / H, src = row * 2u * H + (e - row * H);
        const float g = load_elem(in, i_dtype, src), u = load_elem(in, i_dtype, src + H);
        store_elem(out, o_dtype, e, vai_oracle_epilogue(epilogue, g) * u);
    }
    return 0;
}

/* Threads the parallel loops use from now on.  A launcher may export OMP_NUM_THREADS=1 to its
 * children (torch.distributed.run does); the timed CPU baseline sets the count it reports. */
void vai_oracle_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int vai_oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
