/*
 * CPU oracle for the W2A8 GEMM path, plain C (TEST INFRASTRUCTURE, not product code).
 *
 * A second, independent restatement of the reference's format arithmetic and of the
 * composed GEMM, used by the tests to cross-check the numpy oracle and by the
 * benchmark's CPU-baseline leg.  The product library never links or calls it.
 *
 * Parity status: the format functions are pinned by the reference's known-answer tests
 * (test_matrix_packer.py:5-61, test_quantization.py:108-140) through tests/golden/;
 * the reference holds no GEMM-level vector, so the GEMM level is "unpinned" by the
 * reference itself and anchored on composing its format functions with a dense matmul.
 *
 * Build: make -C oracle      (gcc -O3 -shared -fPIC)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* matrix_packer.py:29-34 : byte = c0<<6 | c1<<4 | c2<<2 | c3 over 4 consecutive columns.
 * Returns 0, or -1 if a value exceeds 3 (matrix_packer.py:20-21), -2 if cols % 4 != 0 (:16-17). */
int oracle_pack_matrix(const uint8_t* codes, int64_t rows, int64_t cols, uint8_t* packed)
{
    if (cols % 4 != 0) return -2;
    for (int64_t i = 0; i < rows * cols; ++i)
        if (codes[i] > 3) return -1;
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t j = 0; j < cols / 4; ++j) {
            const uint8_t* c = codes + r * cols + 4 * j;
            packed[r * (cols / 4) + j] = (uint8_t)((c[0] << 6) | (c[1] << 4) | (c[2] << 2) | c[3]);
        }
    return 0;
}

/* matrix_packer.py:57-64 : codes 4j..4j+3 = byte >> 6,4,2,0 & 3. */
void oracle_unpack_matrix(const uint8_t* packed, int64_t rows, int64_t pcols, uint8_t* codes)
{
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t j = 0; j < pcols; ++j) {
            uint8_t b = packed[r * pcols + j];
            uint8_t* c = codes + r * pcols * 4 + 4 * j;
            c[0] = (b >> 6) & 3; c[1] = (b >> 4) & 3; c[2] = (b >> 2) & 3; c[3] = b & 3;
        }
}

/* IEEE binary16 <-> binary32, round-to-nearest-even (numpy's astype(float16)). */
static float half_to_float(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 1023u, bits;
    if (e == 0) {
        if (m == 0) bits = sign;
        else { int s = 0; while (!(m & 1024u)) { m <<= 1; ++s; } m &= 1023u;
               bits = sign | ((uint32_t)(113 - s) << 23) | (m << 13); }
    } else if (e == 31) bits = sign | 0x7f800000u | (m << 13);
    else bits = sign | ((e + 112u) << 23) | (m << 13);
    float f; memcpy(&f, &bits, 4); return f;
}

static uint16_t float_to_half(float f)
{
    uint32_t x; memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);                 /* NaN */
    if (x >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);                /* >= 65536 -> inf */
    if (x < 0x38800000u) {                                                  /* below 2^-14: half subnormal */
        const uint32_t magic_bits = (uint32_t)((127 - 15) + (23 - 10) + 1) << 23;
        float v, magic; memcpy(&v, &x, 4); memcpy(&magic, &magic_bits, 4);
        v += magic;                                                         /* FPU rounds to nearest even */
        uint32_t r; memcpy(&r, &v, 4);
        return (uint16_t)(sign | (r - magic_bits));
    }
    const uint32_t odd = (x >> 13) & 1u;
    x += ((uint32_t)(15 - 127) << 23) + 0xfffu + odd;                       /* rebias + round half even */
    return (uint16_t)(sign | (x >> 13));
}

/* quantization.py:82-93 : fp16( (fp32(code) - zp) * scale[g, c] ), groups along rows.
 * codes [R, C] u8, scales [R/g, C] fp16 bits, out [R, C] fp16 bits. */
void oracle_dequantize_from_uint2(const uint8_t* codes, const uint16_t* scales, int64_t rows,
                                  int64_t cols, int group_size, int zero_point, uint16_t* out)
{
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c) {
            float s = half_to_float(scales[(r / group_size) * cols + c]);
            out[r * cols + c] = float_to_half(((float)codes[r * cols + c] - (float)zero_point) * s);
        }
}

/* quantization.py:26-46 : scale = max(absmax,1e-9)/1.5 ; code = clip(rint(x/scale)+1, 0, 3).
 * matrix [R, C] double (the reference computes in the input's dtype; tests use float64/float32). */
void oracle_quantize_to_uint2(const double* matrix, int64_t rows, int64_t cols, int group_size,
                              uint8_t* codes, double* scales)
{
    for (int64_t g = 0; g < rows / group_size; ++g)
        for (int64_t c = 0; c < cols; ++c) {
            double amax = 0.0;
            for (int i = 0; i < group_size; ++i) {
                double v = fabs(matrix[(g * group_size + i) * cols + c]);
                if (v > amax) amax = v;
            }
            if (amax < 1e-9) amax = 1e-9;
            double s = amax / 1.5;
            scales[g * cols + c] = s;
            for (int i = 0; i < group_size; ++i) {
                double q = nearbyint(matrix[(g * group_size + i) * cols + c] / s) + 1.0;
                if (q < 0.0) q = 0.0;
                if (q > 3.0) q = 3.0;
                codes[(g * group_size + i) * cols + c] = (uint8_t)q;
            }
        }
}

/* P[g, m, n] = sum_{k in g} x_q[m,k] * (code[n,k] - zp), int32, exact.
 * code from matrix_packer.py:57-64, value from quantization.py:89-90. */
void oracle_w2a8_partials(const int8_t* x_q, const uint8_t* w_packed, int64_t M, int64_t N,
                          int64_t K, int group_size, int zero_point, int32_t* partials)
{
    const int64_t groups = K / group_size;
    for (int64_t n = 0; n < N; ++n) {
        int8_t* w = (int8_t*)malloc((size_t)K);
        for (int64_t j = 0; j < K / 4; ++j) {
            uint8_t b = w_packed[n * (K / 4) + j];
            w[4 * j + 0] = (int8_t)(((b >> 6) & 3) - zero_point);
            w[4 * j + 1] = (int8_t)(((b >> 4) & 3) - zero_point);
            w[4 * j + 2] = (int8_t)(((b >> 2) & 3) - zero_point);
            w[4 * j + 3] = (int8_t)((b & 3) - zero_point);
        }
        for (int64_t m = 0; m < M; ++m)
            for (int64_t g = 0; g < groups; ++g) {
                int32_t acc = 0;
                const int8_t* xr = x_q + m * K + g * group_size;
                const int8_t* wr = w + g * group_size;
                for (int k = 0; k < group_size; ++k) acc += (int32_t)xr[k] * (int32_t)wr[k];
                partials[(g * M + m) * N + n] = acc;
            }
        free(w);
    }
}

/* out[m,n] (fp32) = x_scale[m] * sum_g fp32(w_scale[g,n]) * fp32(P[g,m,n]), g ascending, fmaf. */
void oracle_w2a8_gemm(const int8_t* x_q, const float* x_scale, const uint8_t* w_packed,
                      const uint16_t* w_scale, int64_t M, int64_t N, int64_t K, int group_size,
                      int zero_point, float* out)
{
    const int64_t groups = K / group_size;
    for (int64_t n = 0; n < N; ++n) {
        int8_t* w = (int8_t*)malloc((size_t)K);
        for (int64_t j = 0; j < K / 4; ++j) {
            uint8_t b = w_packed[n * (K / 4) + j];
            w[4 * j + 0] = (int8_t)(((b >> 6) & 3) - zero_point);
            w[4 * j + 1] = (int8_t)(((b >> 4) & 3) - zero_point);
            w[4 * j + 2] = (int8_t)(((b >> 2) & 3) - zero_point);
            w[4 * j + 3] = (int8_t)((b & 3) - zero_point);
        }
        for (int64_t m = 0; m < M; ++m) {
            float acc = 0.0f;
            for (int64_t g = 0; g < groups; ++g) {
                int32_t p = 0;
                const int8_t* xr = x_q + m * K + g * group_size;
                const int8_t* wr = w + g * group_size;
                for (int k = 0; k < group_size; ++k) p += (int32_t)xr[k] * (int32_t)wr[k];
                acc = fmaf(half_to_float(w_scale[g * N + n]), (float)p, acc);
            }
            out[m * N + n] = acc * x_scale[m];
        }
        free(w);
    }
}
