/* Plain-C restatement of the row-parallel hot path's arithmetic. TEST INFRASTRUCTURE ONLY: built by
 * oracle/c/build.py into oracle/c/liboracle.so and loaded by tests/ (and bench.py's CPU legs); the product library
 * never links or calls it.
 *
 * Follows the reference file by file:
 *   orc_reduce, orc_reduce_norm   dlmrt/ops/csrc/tp_comm.cu:216-267 (owner branch), :80-109 (add / pack / block_sum)
 *   orc_gemm_bf16                 dlmrt/layers/linear.py:41-51 with the K order of dlmrt/ops/triton/gemm.py:1-8
 *                                 (FP32 accumulation in increasing K; `splits` K ranges summed in order)
 *   orc_nvfp4_dequant             dlmrt/quantization/nvfp4.py:41-46
 *   orc_nvfp4_down                dlmrt/ops/triton/nvfp4_moe.py:107-131 (_down)
 *   orc_moe_combine               dlmrt/ops/triton/nvfp4_moe.py:134-150 (_combine)
 * Compile with -ffp-contract=off: every fused multiply-add below is written as fmaf on purpose.
 *
 * Parity status: checked against the numpy restatement (oracle/*.py) and, through it, against the reference-made
 * fixtures in tests/golden; the reduction has no reference fixture (see oracle/reduce.py).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static uint16_t f32_to_bf16(float f) { /* cvt.rn.bf16.f32: nearest even, canonical NaN */
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFF;
    return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

/* K1: out[rows, n] = bf16(sum over s of partials[s]) in FP32, rank order, starting from +0.0f. */
void orc_reduce(const uint16_t* partials, int world, int rows, int n, uint16_t* out) {
    const size_t plane = (size_t)rows * n;
    for (size_t i = 0; i < plane; ++i) {
        float v = 0.0f;
        for (int s = 0; s < world; ++s) v += bf16_to_f32(partials[s * plane + i]);
        out[i] = f32_to_bf16(v);
    }
}

static float butterfly32(float* x) { /* x += x[lane ^ o] for o = 16..1; returns lane 0 */
    float y[32];
    for (int o = 16; o > 0; o >>= 1) {
        for (int l = 0; l < 32; ++l) y[l] = x[l] + x[l ^ o];
        memcpy(x, y, sizeof(y));
    }
    return x[0];
}

/* K2 (h == NULL) / K3. h holds `world` copies [world, rows, n]; rank r's own rows of copy r are updated in place. */
void orc_reduce_norm(const uint16_t* partials, uint16_t* h, const uint16_t* weight, float eps, float scale, int world,
                     int rows, int n, uint16_t* out) {
    const size_t plane = (size_t)rows * n;
    const int R = rows / world, threads = n / 8, warps = threads / 32;
    float v[8192], ss[1024], second[32];
    for (int row = 0; row < rows; ++row) {
        const int owner = row / R;
        for (int c = 0; c < n; ++c) {
            float a = 0.0f;
            for (int s = 0; s < world; ++s) a += bf16_to_f32(partials[s * plane + (size_t)row * n + c]);
            a = bf16_to_f32(f32_to_bf16(a)); /* rounded to BF16 before the residual add (tp_comm.cu:238-242) */
            if (h) {
                uint16_t* hp = h + owner * plane + (size_t)row * n + c;
                a += bf16_to_f32(*hp);
                *hp = f32_to_bf16(a);
            }
            v[c] = a;
        }
        for (int t = 0; t < threads; ++t) {
            float acc = 0.0f;
            for (int i = 0; i < 8; ++i) acc = fmaf(v[8 * t + i], v[8 * t + i], acc);
            ss[t] = acc;
        }
        memset(second, 0, sizeof(second));
        for (int w = 0; w < warps; ++w) second[w] = butterfly32(ss + 32 * w);
        const float total = butterfly32(second);
        const float r = (float)(1.0 / sqrt((double)(total / (float)n + eps))) * scale;
        for (int c = 0; c < n; ++c) out[(size_t)row * n + c] = f32_to_bf16(v[c] * r * bf16_to_f32(weight[c]));
    }
}

/* out[m, n] FP32 = x[m, k] * w[n, k]^T, FP32 accumulation in increasing K; `splits` ranges of whole 64-wide k-blocks
 * (range s covers blocks [s*nkb/splits, (s+1)*nkb/splits)), each summed from zero, then added in order. */
void orc_gemm_bf16(const uint16_t* x, const uint16_t* w, int m, int n, int k, int splits, float* out) {
    const int nkb = k / 64;
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) {
            float total = 0.0f;
            for (int s = 0; s < splits; ++s) {
                const int lo = (int)((long long)s * nkb / splits) * 64, hi = (int)((long long)(s + 1) * nkb / splits) * 64;
                float acc = 0.0f;
                for (int c = lo; c < hi; ++c) acc = fmaf(bf16_to_f32(x[(size_t)i * k + c]), bf16_to_f32(w[(size_t)j * k + c]), acc);
                total = s == 0 ? acc : total + acc;
            }
            out[(size_t)i * n + j] = total;
        }
}

void orc_round_bf16(const float* in, size_t count, uint16_t* out) {
    for (size_t i = 0; i < count; ++i) out[i] = f32_to_bf16(in[i]);
}

static const float kE2M1[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

static float e4m3_to_f32(uint8_t b) {
    const int exp = (b >> 3) & 0xF, man = b & 7;
    float v;
    if (exp == 15 && man == 7) return NAN;
    v = exp == 0 ? ldexpf((float)man / 8.0f, -6) : ldexpf(1.0f + (float)man / 8.0f, exp - 7);
    return (b & 0x80) ? -v : v;
}

static float fp4_value(const uint8_t* codes, const uint8_t* scales, int c) {
    const uint8_t byte = codes[c >> 1];
    const uint8_t code = (c & 1) ? (byte >> 4) : (byte & 0xF); /* even element in the low nibble */
    return kE2M1[code] * e4m3_to_f32(scales[c >> 4]);
}

/* [rows, k/2] codes + [rows, k/16] E4M3 scales + per-tensor scale -> [rows, k] BF16. */
void orc_nvfp4_dequant(const uint8_t* codes, const uint8_t* scales, float scale2, int rows, int k, uint16_t* out) {
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < k; ++c) {
            const uint8_t byte = codes[(size_t)r * (k / 2) + (c >> 1)];
            const uint8_t code = (c & 1) ? (byte >> 4) : (byte & 0xF);
            const float s = e4m3_to_f32(scales[(size_t)r * (k / 16) + (c >> 4)]) * scale2;
            out[(size_t)r * k + c] = f32_to_bf16(kE2M1[code] * s);
        }
}

/* GEMM2 of one expert: y[m, n] = bf16((sum over f of a[m, f] * w[n, f]) * g2), FP32 in increasing f. */
void orc_nvfp4_down(const uint8_t* a_codes, const uint8_t* a_scales, const uint8_t* w_codes, const uint8_t* w_scales,
                    float g2, int m, int n, int f, uint16_t* y) {
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) {
            float acc = 0.0f;
            for (int c = 0; c < f; ++c)
                acc = fmaf(fp4_value(a_codes + (size_t)i * (f / 2), a_scales + (size_t)i * (f / 16), c),
                           fp4_value(w_codes + (size_t)j * (f / 2), w_scales + (size_t)j * (f / 16), c), acc);
            y[(size_t)i * n + j] = f32_to_bf16(acc * g2);
        }
}

/* out[rows, n] = bf16(sum over k in list order of (local ? weight : 0) * y[row * top_k + k]) [+ shared -> bf16]. */
void orc_moe_combine(const uint16_t* y, const int32_t* ids, const float* weights, const uint16_t* shared, int lo,
                     int local, int rows, int top_k, int n, uint16_t* out) {
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < n; ++c) {
            float acc = 0.0f;
            for (int k = 0; k < top_k; ++k) {
                const int e = ids[r * top_k + k] - lo;
                const int is_local = e >= 0 && e < local;
                const float yv = is_local ? bf16_to_f32(y[((size_t)r * top_k + k) * n + c]) : 0.0f;
                acc = fmaf(is_local ? weights[r * top_k + k] : 0.0f, yv, acc);
            }
            uint16_t o = f32_to_bf16(acc);
            if (shared) o = f32_to_bf16(bf16_to_f32(o) + bf16_to_f32(shared[(size_t)r * n + c]));
            out[(size_t)r * n + c] = o;
        }
}
