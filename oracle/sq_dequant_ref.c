/*
 * CPU oracle for the SquareQ INT8 -> floating-point weight dequant.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA path is
 * compared against (tests, the smoke check and the benchmark's CPU-baseline
 * leg).  Nothing in the shipped package links, imports or calls it.
 *
 * It restates, in scalar C, the arithmetic of the reference's host dequant
 * (src/stagehand/scheduler.py:290-300):
 *
 *     q2d      = qweight.reshape(rows_stored, -1)[:out, :in]
 *     scale    = scale.reshape(-1).float()[:out]
 *     zero     = zero_point.reshape(-1).float()[:out]
 *     dequant  = (q2d.float() - zero[:, None]) * scale[:, None]
 *     dst      = dequant.to(runtime_dtype)
 *
 * i.e. per element:  x = (float)q  (exact);  y = x - zp  (one fp32 rounding);
 * w = y * s (one fp32 rounding);  out = round-to-nearest-even(w) in the
 * runtime dtype.  The two fp32 operations are kept as two separately rounded
 * operations (build with -ffp-contract=off; see the Makefile).
 *
 * The bias / small-parameter cast restates `bias.to(dtype)` and
 * `param.data.to(dtype)` (src/stagehand/scheduler.py:305, :313).
 *
 * The fp32 -> bf16 rounding follows the published algorithm of the third-party
 * dependency that performs it in the reference (torch >= 2.1.0, pinned only by
 * pyproject.toml:27; c10::BFloat16 round-to-nearest-even: add 0x7FFF plus the
 * LSB of the kept half, then truncate).  NaN inputs produce 0x7FC0 here; the
 * reference's vectorised and scalar loops emit different NaN payloads, so
 * parity on NaN is "NaN in the same positions", not a bit pattern.
 *
 * Parity pin: checked bit-for-bit against outputs of the reference's own
 * `_copy_squareq_backed_params_into_buffer` captured in tests/golden/
 * (see tests/golden/make_golden.py).
 */
#include <stdint.h>
#include <string.h>
#include <stddef.h>

enum { SQ_REF_OUT_BF16 = 0, SQ_REF_OUT_F16 = 1, SQ_REF_OUT_F32 = 2 };

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* fp32 -> bf16, round to nearest even. */
uint16_t sq_ref_f32_to_bf16(float f)
{
    uint32_t u = f32_bits(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FC0u;         /* NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7FFFu + lsb;
    return (uint16_t)(u >> 16);
}

/* fp32 -> IEEE binary16, round to nearest even, subnormals kept. */
uint16_t sq_ref_f32_to_f16(float f)
{
    uint32_t u = f32_bits(f);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t mag = u & 0x7FFFFFFFu;
    if (mag > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);   /* NaN */
    if (mag >= 0x47800000u) {                                    /* >= 65536: Inf (or overflow after rounding handled below) */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (mag < 0x38800000u) {                                     /* < 2^-14: subnormal half or zero */
        if (mag < 0x33000000u) return (uint16_t)sign;            /* < 2^-25 rounds to 0 */
        /* value = m * 2^-24 with m in [0, 1024]; compute via fp32 add of 0.5 (exact RNE trick) */
        float a = bits_f32(mag);
        float magic = bits_f32(0x3F000000u);                     /* 0.5f */
        float r = a + magic;                                     /* low mantissa bits now hold the rounded m (RNE) */
        uint32_t m = f32_bits(r) - 0x3F000000u;
        return (uint16_t)(sign | m);
    }
    /* normal half */
    uint32_t lsb = (mag >> 13) & 1u;
    mag += 0xFFFu + lsb;                                         /* RNE on the 13 dropped bits */
    uint32_t h = (mag - 0x38000000u) >> 13;                      /* rebias exponent 127 -> 15 */
    if (h >= 0x7C00u) h = 0x7C00u;                               /* rounded up to Inf */
    return (uint16_t)(sign | h);
}

static inline void store_out(void *dst, int64_t i, float w, int out_dtype)
{
    if (out_dtype == SQ_REF_OUT_BF16)      ((uint16_t *)dst)[i] = sq_ref_f32_to_bf16(w);
    else if (out_dtype == SQ_REF_OUT_F16)  ((uint16_t *)dst)[i] = sq_ref_f32_to_f16(w);
    else                                   ((float *)dst)[i] = w;
}

/*
 * Dequantise a [rows, cols] window of an int8 matrix stored with row stride
 * `ld` (>= cols; this is the slab's padded_in_features) into a dense
 * [rows, cols] destination.  scale and zero_point have one fp32 entry per row.
 * zero_point may be NULL (treated as +0.0, which is bit-identical because
 * (float)q - 0.0f == (float)q for every int8 q).
 * Follows src/stagehand/scheduler.py:290-300.
 */
void sq_ref_dequant_rows(const int8_t *q, int64_t ld,
                         const float *scale, const float *zero_point,
                         int64_t rows, int64_t cols,
                         void *dst, int out_dtype)
{
    for (int64_t r = 0; r < rows; ++r) {
        const int8_t *qr = q + r * ld;
        volatile float s = scale[r];
        volatile float z = zero_point ? zero_point[r] : 0.0f;
        for (int64_t c = 0; c < cols; ++c) {
            volatile float x = (float)qr[c];
            volatile float y = x - z;          /* first fp32 rounding  */
            volatile float w = y * s;          /* second fp32 rounding */
            store_out(dst, r * cols + c, w, out_dtype);
        }
    }
}

/* fp32 -> runtime dtype cast of a flat vector (bias and module-owned params). */
void sq_ref_cast_f32(const float *src, int64_t n, void *dst, int out_dtype)
{
    for (int64_t i = 0; i < n; ++i) store_out(dst, i, src[i], out_dtype);
}

/*
 * Same arithmetic without the volatile fences, split over rows so several
 * host threads can run it.  Used only by the benchmark's CPU-baseline leg to
 * time a tight single-pass host dequant; validated against sq_ref_dequant_rows.
 */
void sq_ref_dequant_rows_fast(const int8_t *q, int64_t ld,
                              const float *scale, const float *zero_point,
                              int64_t row_begin, int64_t row_end, int64_t cols,
                              void *dst, int out_dtype)
{
    for (int64_t r = row_begin; r < row_end; ++r) {
        const int8_t *qr = q + r * ld;
        const float s = scale[r];
        const float z = zero_point ? zero_point[r] : 0.0f;
        if (out_dtype == SQ_REF_OUT_BF16) {
            uint16_t *o = (uint16_t *)dst + r * cols;
            for (int64_t c = 0; c < cols; ++c) {
                float w = ((float)qr[c] - z) * s;
                uint32_t u = f32_bits(w);
                uint32_t rounded = (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
                o[c] = ((u & 0x7FFFFFFFu) > 0x7F800000u) ? (uint16_t)0x7FC0u : (uint16_t)rounded;
            }
        } else {
            for (int64_t c = 0; c < cols; ++c)
                store_out(dst, r * cols + c, ((float)qr[c] - z) * s, out_dtype);
        }
    }
}
