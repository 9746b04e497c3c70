/* TEST INFRASTRUCTURE ONLY - plain-C CPU oracle for the quantized matvec path.
 *
 * Restates the reference's block decoders (engine/csrc/common/qwen_quant.cuh:151-279, the CUDA
 * twin of engine/src/vinf/gguf/dequant.py:121-500) one whole block at a time, then does the
 * contraction in double precision (engine/src/vinf/reference_ops.py:18-32) and the row argmax with
 * the reference's tie rule (engine/csrc/megakernel/qwen_runtime.cu:851-876).
 *
 * Parity status: PINNED through oracle/dequant_np.py - tests/test_oracle_golden.py requires this
 * library to return bit-identical values to the numpy oracle, which is itself checked against the
 * reference's known-answer vectors and against outputs of the reference dequantiser.
 *
 * Only tests, the smoke check and the benchmark's CPU-baseline leg may load this library.
 * Build: make -C oracle   (gcc -O2 -fopenmp -fPIC -shared).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { T_F32 = 0, T_F16 = 1, T_Q8_0 = 8, T_Q2_K = 10, T_Q3_K = 11, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14,
       T_IQ2_XXS = 16, T_IQ2_XS = 17, T_IQ3_XXS = 18, T_IQ4_NL = 20, T_IQ3_S = 21, T_IQ2_S = 22, T_IQ4_XS = 23 };

/* qwen_quant.cuh:40-58 */
int oracle_traits(int type, int *block, int *size) {
    switch (type) {
        case T_F32: *block = 1; *size = 4; return 1;
        case T_F16: *block = 1; *size = 2; return 1;
        case T_Q8_0: *block = 32; *size = 34; return 1;
        case T_Q2_K: *block = 256; *size = 84; return 1;
        case T_Q3_K: *block = 256; *size = 110; return 1;
        case T_Q4_K: *block = 256; *size = 144; return 1;
        case T_Q5_K: *block = 256; *size = 176; return 1;
        case T_Q6_K: *block = 256; *size = 210; return 1;
        case T_IQ4_NL: *block = 32; *size = 18; return 1;
        case T_IQ3_S: *block = 256; *size = 110; return 1;
        case T_IQ4_XS: *block = 256; *size = 136; return 1;
        case T_IQ2_XXS: *block = 256; *size = 66; return 1;
        case T_IQ2_XS: *block = 256; *size = 74; return 1;
        case T_IQ2_S: *block = 256; *size = 82; return 1;
        case T_IQ3_XXS: *block = 256; *size = 98; return 1;
        default: return 0;
    }
}

static const int kIq4Levels[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

/* IEEE half -> double, by hand so that the oracle needs no F16C. */
static double half_at(const uint8_t *p) {
    const unsigned h = p[0] | (p[1] << 8);
    const int sign = h >> 15, e = (h >> 10) & 31, m = h & 1023;
    double v;
    if (e == 0) v = ldexp((double)m, -24);
    else if (e == 31) v = m ? NAN : INFINITY;
    else v = ldexp((double)(m | 1024), e - 25);
    return sign ? -v : v;
}

static uint32_t le32(const uint8_t *p) { return p[0] | (p[1] << 8) | (p[2] << 16) | ((uint32_t)p[3] << 24); }

/* Sign byte of 7 stored bits: the eighth bit restores even parity (table c_ksigns_iq2xs). */
static int ksign(int i) {
    int p = 0;
    for (int b = 0; b < 7; ++b) p ^= (i >> b) & 1;
    return i | (p << 7);
}

static void k4_pair(const uint8_t *s, int g, int *sc, int *mn) { /* qwen_quant.cuh:78-86 */
    if (g < 4) { *sc = s[g] & 63; *mn = s[g + 4] & 63; }
    else { *sc = (s[g + 4] & 15) | ((s[g - 4] >> 6) << 4); *mn = (s[g + 4] >> 4) | ((s[g] >> 6) << 4); }
}

/* One block -> `block` doubles.  All products are exact in double; each result is then exactly
 * the value the reference computes (and is representable in fp32 for finite fp16 scales). */
static void decode_block(int type, const uint8_t *b, double *o, const uint8_t *grid) {
    switch (type) {
    case T_Q8_0: { /* :154-158 */
        const double d = half_at(b);
        for (int i = 0; i < 32; ++i) o[i] = d * (int8_t)b[2 + i];
    } break;
    case T_IQ4_NL: { /* :159-164 */
        const double d = half_at(b);
        for (int i = 0; i < 32; ++i) o[i] = d * kIq4Levels[i < 16 ? b[2 + i] & 15 : b[2 + i - 16] >> 4];
    } break;
    case T_Q4_K: case T_Q5_K: { /* :165-181 */
        const double d = half_at(b), dmin = half_at(b + 2);
        const uint8_t *qh = b + 16, *qs = type == T_Q4_K ? b + 16 : b + 48;
        for (int g = 0; g < 8; ++g) {
            int sc, mn;
            k4_pair(b + 4, g, &sc, &mn);
            const double dl = d * sc, ml = dmin * mn;
            for (int i = 0; i < 32; ++i) {
                int q = (qs[32 * (g / 2) + i] >> (4 * (g % 2))) & 15;
                if (type == T_Q5_K) q += ((qh[i] >> g) & 1) << 4;
                o[32 * g + i] = dl * q - ml;
            }
        }
    } break;
    case T_Q6_K: { /* :182-190 */
        const double d = half_at(b + 208);
        for (int e = 0; e < 256; ++e) {
            const int chunk = e / 128, quarter = (e % 128) / 32, l = e % 32;
            const int lo = (b[chunk * 64 + (quarter % 2) * 32 + l] >> (quarter >= 2 ? 4 : 0)) & 15;
            const int hi = (b[128 + chunk * 32 + l] >> (2 * quarter)) & 3;
            o[e] = d * (int8_t)b[192 + e / 16] * ((lo | (hi << 4)) - 32);
        }
    } break;
    case T_Q2_K: { /* :191-198 */
        const double d = half_at(b + 80), dmin = half_at(b + 82);
        for (int e = 0; e < 256; ++e) {
            const int sc = b[e / 16];
            const int q = (b[16 + 32 * (e / 128) + e % 32] >> (2 * ((e % 128) / 32))) & 3;
            o[e] = d * (sc & 15) * q - dmin * (sc >> 4);
        }
    } break;
    case T_Q3_K: { /* :199-210 */
        const double d = half_at(b + 108);
        const uint8_t *s = b + 96;
        for (int e = 0; e < 256; ++e) {
            const int k = e / 16;
            const int scale = (((s[k % 8] >> (4 * (k / 8))) & 15) | (((s[8 + k % 4] >> (2 * (k / 4))) & 3) << 4)) - 32;
            const int low = (b[32 + 32 * (e / 128) + e % 32] >> (2 * ((e % 128) / 32))) & 3;
            const int q = low - (((b[e % 32] >> (e / 32)) & 1) ? 0 : 4);
            o[e] = d * scale * q;
        }
    } break;
    case T_IQ4_XS: { /* :211-220 */
        const double d = half_at(b);
        const int scales_h = b[2] | (b[3] << 8);
        for (int g = 0; g < 8; ++g) {
            const int ls = ((b[4 + g / 2] >> (4 * (g % 2))) & 15) | (((scales_h >> (2 * g)) & 3) << 4);
            const double dl = d * (ls - 32);
            for (int i = 0; i < 32; ++i)
                o[32 * g + i] = dl * kIq4Levels[i < 16 ? b[8 + 16 * g + i] & 15 : b[8 + 16 * g + i - 16] >> 4];
        }
    } break;
    case T_IQ3_S: { /* :221-234 */
        const double d = half_at(b);
        for (int e = 0; e < 256; ++e) {
            const int g = e / 32, idx = e / 4;
            const double db = d * (1 + 2 * ((b[106 + g / 2] >> (4 * (g % 2))) & 15));
            const int entry = b[2 + idx] | (((b[66 + idx / 8] >> (idx % 8)) & 1) << 8);
            const int neg = (b[74 + e / 8] >> (e % 8)) & 1;
            o[e] = db * grid[entry * 4 + e % 4] * (neg ? -1.0 : 1.0);
        }
    } break;
    case T_IQ2_XXS: { /* :235-258 */
        const double d = half_at(b);
        for (int ib = 0; ib < 8; ++ib) {
            const uint32_t aux1 = le32(b + 2 + 8 * ib + 4);
            const double db = d * (0.5 + (aux1 >> 28)) * 0.25;
            for (int l = 0; l < 4; ++l) {
                const uint8_t *g = grid + 8 * b[2 + 8 * ib + l];
                const int signs = ksign((aux1 >> (7 * l)) & 127);
                for (int j = 0; j < 8; ++j) o[32 * ib + 8 * l + j] = db * g[j] * (((signs >> j) & 1) ? -1.0 : 1.0);
            }
        }
    } break;
    case T_IQ2_XS: {
        const double d = half_at(b);
        for (int ib = 0; ib < 8; ++ib)
            for (int l = 0; l < 4; ++l) {
                const int q = b[2 + 2 * (4 * ib + l)] | (b[3 + 2 * (4 * ib + l)] << 8);
                const double db = d * (0.5 + ((b[66 + ib] >> (4 * (l / 2))) & 15)) * 0.25;
                const uint8_t *g = grid + 8 * (q & 511);
                const int signs = ksign(q >> 9);
                for (int j = 0; j < 8; ++j) o[32 * ib + 8 * l + j] = db * g[j] * (((signs >> j) & 1) ? -1.0 : 1.0);
            }
    } break;
    case T_IQ2_S: {
        const double d = half_at(b);
        for (int ib = 0; ib < 8; ++ib)
            for (int l = 0; l < 4; ++l) {
                const int entry = b[2 + 4 * ib + l] | ((b[66 + ib] << (8 - 2 * l)) & 0x300);
                const int signs = b[34 + 4 * ib + l];
                const double db = d * (0.5 + ((b[74 + ib] >> (4 * (l / 2))) & 15)) * 0.25;
                const uint8_t *g = grid + 8 * entry;
                for (int j = 0; j < 8; ++j) o[32 * ib + 8 * l + j] = db * g[j] * (((signs >> j) & 1) ? -1.0 : 1.0);
            }
    } break;
    case T_IQ3_XXS: { /* :259-270 */
        const double d = half_at(b);
        for (int ib = 0; ib < 8; ++ib) {
            const uint32_t aux = le32(b + 66 + 4 * ib);
            const double db = d * (0.5 + (aux >> 28)) * 0.5;
            for (int l = 0; l < 4; ++l) {
                const int signs = ksign((aux >> (7 * l)) & 127);
                for (int h = 0; h < 2; ++h) {
                    const uint8_t *g = grid + 4 * b[2 + 8 * ib + 2 * l + h];
                    for (int j = 0; j < 4; ++j)
                        o[32 * ib + 8 * l + 4 * h + j] = db * g[j] * (((signs >> (4 * h + j)) & 1) ? -1.0 : 1.0);
                }
            }
        }
    } break;
    case T_F32: { float f; memcpy(&f, b, 4); o[0] = f; } break;
    case T_F16: o[0] = half_at(b); break;
    }
}

/* Dequantise rows x cols weights into `out` (doubles). Returns 0, or -1 for a bad type/shape. */
int oracle_dequantize(int type, const uint8_t *w, long rows, int cols, double *out, const uint8_t *grid) {
    int block, size;
    if (!oracle_traits(type, &block, &size) || cols <= 0 || cols % block) return -1;
    const long nblk = rows * (cols / block);
#pragma omp parallel for schedule(static)
    for (long i = 0; i < nblk; ++i) decode_block(type, w + i * size, out + i * block, grid);
    return 0;
}

/* y[t * rows + r] = sum_k W[r][k] x[t * cols + k], accumulated in double in column order. */
int oracle_qmv(int type, const uint8_t *w, int rows, int cols, const float *x, int ntok, double *y,
               const uint8_t *grid) {
    int block, size;
    if (!oracle_traits(type, &block, &size) || cols <= 0 || cols % block || ntok < 1) return -1;
    const size_t row_bytes = (size_t)(cols / block) * size;
#pragma omp parallel
    {
        double *wr = malloc(sizeof(double) * cols);
#pragma omp for schedule(static)
        for (int r = 0; r < rows; ++r) {
            for (int k = 0; k < cols / block; ++k)
                decode_block(type, w + r * row_bytes + (size_t)k * size, wr + (size_t)k * block, grid);
            for (int t = 0; t < ntok; ++t) {
                const float *xt = x + (size_t)t * cols;
                double acc = 0.0;
                for (int k = 0; k < cols; ++k) acc += wr[k] * xt[k];
                y[(size_t)t * rows + r] = acc;
            }
        }
        free(wr);
    }
    return 0;
}

/* Row-wise argmax of [ntok][n] logits: strict '>' scan from -inf, lowest index wins ties, a row
 * with nothing above -inf (all -inf or NaN) gives 0x7fffffff (qwen_runtime.cu:851-876). */
void oracle_argmax_rows(const double *y, int n, int ntok, int *out) {
    for (int t = 0; t < ntok; ++t) {
        double best = -INFINITY;
        int idx = 0x7fffffff;
        for (int i = 0; i < n; ++i)
            if (y[(size_t)t * n + i] > best) { best = y[(size_t)t * n + i]; idx = i; }
        out[t] = idx;
    }
}
