/*
 * espdl_oracle.c - TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C, single-threaded restatement of the arithmetic of ESP-DL's
 * generic ("ANSI C") quantized operators, written as straightforward loops
 * over the same descriptor structs the CUDA backend's C ABI takes (with HOST
 * pointers here).  It exists only so that tests, the smoke check and the
 * benchmark's cpu_baseline leg can compare the CUDA kernels against an
 * independent implementation; the shipped library never links or calls it.
 *
 * Pinning: every function here is cross-checked (tests/test_oracle_vs_reference.py)
 * against the reference's own C++ operators compiled unmodified from its
 * source tree (oracle/ref_harness.cpp -> oracle/_ref/libespdl_ref.so) and
 * against the reference's shipped golden Gemm / MLP vectors (tests/golden/).
 * The only semantics with no compiled reference counterpart are the
 * per-channel filter exponents (the reference's C epilogue has no working
 * per-channel branch; the rule restated here is the ESP32-P4 assembly one,
 * see oracle_requant below) and the batch extent n > 1 (the reference reads
 * one image; here image i is an independent repetition of the same op).
 *
 * Each function cites the reference file:line (paths relative to the
 * reference project root) whose behaviour it restates.
 */
#include "../include/espdl_b200.h"

#include <limits.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#if defined(_OPENMP)
#include <omp.h>
#endif

/* ------------------------------------------------------------ primitives */

/* dl::tool::truncate  esp-dl/dl/tool/include/dl_tool.hpp:225-254 */
static inline int64_t clamp64(int64_t v, int64_t lo, int64_t hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* dl::tool::round(float): (int)floorf(value + 0.5) with a double literal, i.e. the
 * sum is formed in double, narrowed to float, then floored.
 * esp-dl/dl/tool/src/dl_tool.cpp:72-90.  Half-even variant: :33-70. */
static inline int fround_half_up(float v) { return (int)floorf((float)((double)v + 0.5)); }

/* Half-even: what ESP32-P4 does (fcvt.w.s with rne, esp-dl/dl/tool/src/dl_tool.cpp:24-31). */
static inline int fround_half_even(float v) { return (int)rintf(v); }

static inline int fround(float v, int mode) { return mode == ESPDL_ROUND_HALF_EVEN ? fround_half_even(v) : fround_half_up(v); }

/* dl::tool::shift_and_round  esp-dl/dl/tool/src/dl_tool.cpp:95-146.
 * shift > 0: arithmetic right shift with half-up or half-even rounding;
 * shift <= 0: left shift in 64 bits, then saturate to the accumulator type
 * (acc_bits = 32 for int8 ops, 64 for int16 ops). */
static inline int64_t shift_and_round(int64_t v, int shift, int mode, int acc_bits)
{
    if (shift <= 0) {
        int64_t s = (int64_t)((uint64_t)v << (-shift));
        if (acc_bits == 32)
            s = clamp64(s, INT32_MIN, INT32_MAX);
        return s;
    }
    if (mode == ESPDL_ROUND_HALF_EVEN) {
        int64_t q = v >> shift;
        int64_t rem = v & (((int64_t)1 << shift) - 1);
        int64_t half = (int64_t)1 << (shift - 1);
        if (rem > half || (rem == half && (q & 1)))
            q += 1;
        return q;
    }
    return (v + ((int64_t)1 << (shift - 1))) >> shift;
}

/* DL_SCALE / DL_RESCALE  esp-dl/dl/dl_define.hpp:84-90 (float power of two) */
static inline float dl_scale(int e) { return e > 0 ? (float)(1 << e) : (float)1.0 / (float)(1 << -e); }
static inline float dl_rescale(int e) { return e > 0 ? (float)1.0 / (float)(1 << e) : (float)(1 << -e); }

/*
 * Conv / depthwise epilogue.
 * per-tensor: esp-dl/dl/base/dl_base_activate_buffer.hpp:27-37,60-73
 *   acc += bias; acc = shift_and_round(acc, mac_shift); relu; truncate.
 * per-channel (no working C branch in the reference; this is the ESP32-P4 rule:
 *   bias pre-loaded into the accumulator esp-dl/dl/base/isa/esp32p4/dl_esp32p4_s8.S:6-11,
 *   shift[c] = e_out - e_w[c] - e_in esp-dl/dl/base/dl_base.hpp:249-252,
 *   shift/round/saturate :57-65, then ReLU dl_esp32p4_s8_conv2d.S:1261-1266).
 * Saturate-then-ReLU equals ReLU-then-saturate, so one code path serves both.
 */
static inline int64_t oracle_requant(int64_t acc, int64_t bias, int shift, int act, int mode, int is16)
{
    if (!is16)
        acc = (int32_t)((uint32_t)(int32_t)acc + (uint32_t)(int32_t)bias); /* 32-bit accumulator wraps */
    else
        acc += bias;
    int64_t v = shift_and_round(acc, shift, mode, is16 ? 64 : 32);
    if (act == ESPDL_ACT_RELU && v < 0)
        v = 0;
    return is16 ? clamp64(v, INT16_MIN, INT16_MAX) : clamp64(v, INT8_MIN, INT8_MAX);
}

static int conv_check(const espdl_conv_desc *d)
{
    if (!d || !d->input || !d->filter || !d->output)
        return ESPDL_ERR_INVALID_ARG;
    if (d->dtype != ESPDL_DTYPE_INT8 && d->dtype != ESPDL_DTYPE_INT16)
        return ESPDL_ERR_UNSUPPORTED;
    if (d->n < 0 || d->in_h <= 0 || d->in_w <= 0 || d->in_c <= 0 || d->out_c <= 0 || d->kh <= 0 || d->kw <= 0)
        return ESPDL_ERR_INVALID_ARG;
    if (d->group != 1 && !(d->group == d->in_c && d->out_c == d->in_c))
        return ESPDL_ERR_UNSUPPORTED;
    if (d->per_channel && !d->filter_exponents)
        return ESPDL_ERR_INVALID_ARG;
    if (d->activation != ESPDL_ACT_LINEAR && d->activation != ESPDL_ACT_RELU)
        return ESPDL_ERR_UNSUPPORTED;
    if (d->residual && (d->dtype != ESPDL_DTYPE_INT8 || d->group != 1))
        return ESPDL_ERR_UNSUPPORTED;
    return ESPDL_OK;
}

/*
 * Conv2D / Gemm / depthwise.
 * MAC loops: esp-dl/dl/base/dl_base_conv2d.cpp:141-162 (conv2d_hwcn, filter [N][H][W][C]),
 *            esp-dl/dl/base/dl_base_depthwise_conv2d.cpp:47-66 (filter [H][W][C]);
 * border handling (skip taps outside the image): esp-dl/dl/base/dl_base.hpp:951-1022;
 * output extents: esp-dl/dl/module/include/dl_module_conv.hpp:81-102.
 */
int oracle_conv2d(const espdl_conv_desc *d)
{
    int st = conv_check(d);
    if (st)
        return st;
    const int is16 = d->dtype == ESPDL_DTYPE_INT16;
    const int ips = d->in_pixel_stride ? d->in_pixel_stride : d->in_c;
    const int ops = d->out_pixel_stride ? d->out_pixel_stride : d->out_c;
    const int dw = d->group != 1;
    const int8_t *in8 = (const int8_t *)d->input;
    const int16_t *in16 = (const int16_t *)d->input;
    const int8_t *w8 = (const int8_t *)d->filter;
    const int16_t *w16 = (const int16_t *)d->filter;
    const int32_t *b32 = (const int32_t *)d->bias;
    const int64_t *b64 = (const int64_t *)d->bias;
    int8_t *o8 = (int8_t *)d->output;
    int16_t *o16 = (int16_t *)d->output;
    const int64_t total_rows = (int64_t)d->n * d->out_h;

#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
    for (int64_t row = 0; row < total_rows; row++) {
        const int n = (int)(row / d->out_h), oy = (int)(row % d->out_h);
        for (int ox = 0; ox < d->out_w; ox++) {
            for (int oc = 0; oc < d->out_c; oc++) {
                int64_t acc = 0;
                for (int ky = 0; ky < d->kh; ky++) {
                    const int iy = oy * d->stride_h + ky * d->dilation_h - d->pad_top;
                    if (iy < 0 || iy >= d->in_h)
                        continue;
                    for (int kx = 0; kx < d->kw; kx++) {
                        const int ix = ox * d->stride_w + kx * d->dilation_w - d->pad_left;
                        if (ix < 0 || ix >= d->in_w)
                            continue;
                        const int64_t ibase = (((int64_t)n * d->in_h + iy) * d->in_w + ix) * ips;
                        if (dw) {
                            const int64_t wi = ((int64_t)ky * d->kw + kx) * d->in_c + oc;
                            acc += is16 ? (int64_t)in16[ibase + oc] * w16[wi] : (int64_t)in8[ibase + oc] * w8[wi];
                        } else {
                            /* filter_image_stride != 0: every image has its own filter (a batch of matrix products) */
                            const int64_t wbase = (int64_t)n * d->filter_image_stride + (((int64_t)oc * d->kh + ky) * d->kw + kx) * d->in_c;
                            if (is16) {
                                for (int c = 0; c < d->in_c; c++) acc += (int64_t)in16[ibase + c] * w16[wbase + c];
                            } else {
                                int32_t a = 0;
                                for (int c = 0; c < d->in_c; c++) a += (int32_t)in8[ibase + c] * w8[wbase + c];
                                acc += a;
                            }
                        }
                    }
                }
                if (!is16)
                    acc = (int32_t)acc;
                const int ew = d->per_channel ? d->filter_exponents[oc] : d->filter_exponent;
                const int shift = d->out_exponent - ew - d->in_exponent;
                const int64_t bias = d->bias ? (is16 ? b64[oc] : (int64_t)b32[oc]) : 0;
                int64_t q = oracle_requant(acc, bias, shift, d->activation, d->round_mode, is16);
                const int64_t oi = (((int64_t)n * d->out_h + oy) * d->out_w + ox) * ops + oc;
                if (is16) {
                    o16[oi] = (int16_t)q;
                } else {
                    /* fused dl::module::LUT node: esp-dl/dl/base/dl_base_lut.cpp:10-15 */
                    int32_t r8 = d->lut ? d->lut[(int64_t)oc * d->lut_channel_stride + ((uint8_t)(int8_t)q ^ 0x80u)] : (int8_t)q;
                    if (d->residual) { /* a following Add with equal exponents: saturating sum, dl_base_add.cpp:8-44 */
                        const int rps = d->residual_pixel_stride ? d->residual_pixel_stride : d->out_c;
                        r8 += ((const int8_t *)d->residual)[(((int64_t)n * d->out_h + oy) * d->out_w + ox) * rps + oc];
                        r8 = r8 > 127 ? 127 : (r8 < -128 ? -128 : r8);
                    }
                    o8[oi] = (int8_t)r8;
                }
            }
        }
    }
    return ESPDL_OK;
}

/* --------------------------------------------------------- elementwise */

static inline int64_t load_int(const void *p, int dtype, int64_t i)
{
    return dtype == ESPDL_DTYPE_INT8 ? ((const int8_t *)p)[i] : ((const int16_t *)p)[i];
}

static inline void store_sat(void *p, int dtype, int64_t i, int64_t v)
{
    if (dtype == ESPDL_DTYPE_INT8)
        ((int8_t *)p)[i] = (int8_t)clamp64(v, INT8_MIN, INT8_MAX);
    else if (dtype == ESPDL_DTYPE_BOOL)
        ((uint8_t *)p)[i] = v != 0;
    else
        ((int16_t *)p)[i] = (int16_t)clamp64(v, INT16_MIN, INT16_MAX);
}

/* quantize<RT>(float, inv_scale): esp-dl/dl/tensor/src/dl_tensor_base.cpp:18-30 */
static inline int64_t quantize_f(float x, float inv_scale, int mode) { return fround(x * inv_scale, mode); }

int oracle_eltwise(const espdl_eltwise_desc *d)
{
    if (!d || !d->input0 || !d->output || d->ndim < 1 || d->ndim > 4)
        return ESPDL_ERR_INVALID_ARG;
    int os[4] = {1, 1, 1, 1}, s0[4] = {1, 1, 1, 1}, s1[4] = {1, 1, 1, 1};
    for (int i = 0; i < d->ndim; i++) {
        os[4 - d->ndim + i] = d->out_shape[i];
        s0[4 - d->ndim + i] = d->in0_shape[i];
        s1[4 - d->ndim + i] = d->in1_shape[i];
    }
    const int binary = d->op == ESPDL_ELT_ADD || d->op == ESPDL_ELT_MUL || d->op == ESPDL_ELT_SUB ||
        (d->op >= ESPDL_ELT_MAX && d->op <= ESPDL_ELT_POW);
    if ((binary || d->op == ESPDL_ELT_LUT || d->op == ESPDL_ELT_PRELU) && !d->input1)
        return ESPDL_ERR_INVALID_ARG;
    int64_t st0[4], st1[4];
    {
        int64_t a = 1, b = 1;
        for (int i = 3; i >= 0; i--) {
            if (s0[i] != os[i] && s0[i] != 1)
                return ESPDL_ERR_INVALID_ARG;
            if (binary && s1[i] != os[i] && s1[i] != 1)
                return ESPDL_ERR_INVALID_ARG;
            st0[i] = s0[i] == 1 ? 0 : a;
            st1[i] = s1[i] == 1 ? 0 : b;
            a *= s0[i];
            b *= s1[i];
        }
    }
    const int mode = d->round_mode;
    const int idt = d->in_dtype, odt = d->out_dtype;
    /* Mul: esp-dl/dl/base/dl_base_mul.cpp:128 - scale = (2^e0 * 2^e1) * 2^-eo, in that float order */
    const float mul_scale = dl_scale(d->in0_exponent) * dl_scale(d->in1_exponent) * dl_rescale(d->out_exponent);
    /* Clip: esp-dl/dl/module/include/dl_module_clip.hpp:85 */
    const float clip_rescale = dl_scale(d->in0_exponent) * dl_rescale(d->out_exponent);
    const int C = os[3];
    /* Div: esp-dl/dl/base/dl_base_div.cpp:66 (scale), :208-250 (which loop body runs: chosen by the operand that is a
     * scalar along the innermost merged axis, esp-dl/dl/base/dl_base_elemwise.cpp:38-100 - the innermost axis on which
     * the output is longer than 1; int8 asks for the dividend first, int16 for the divisor first), :17-31 (an int8
     * dividend of one element is tabulated by divisor, which differs from the loop body at 0 / 0). */
    int div_n1 = 0, div_table0 = 0;
    float div_scale = 0;
    if (d->op == ESPDL_ELT_DIV) {
        int ax = 3;
        while (ax > 0 && os[ax] == 1) ax--;
        const int in0_1 = s0[ax] == 1, in1_1 = s1[ax] == 1;
        div_table0 = idt == ESPDL_DTYPE_INT8 && (int64_t)s0[0] * s0[1] * s0[2] * s0[3] == 1;
        div_n1 = idt == ESPDL_DTYPE_INT8 ? (in1_1 && !in0_1) : in1_1;
        div_scale = dl_rescale(d->out_exponent) * dl_scale(d->in0_exponent) / dl_scale(d->in1_exponent);
    }
    int64_t oi = 0;
    for (int i3 = 0; i3 < os[0]; i3++)
        for (int i2 = 0; i2 < os[1]; i2++)
            for (int i1 = 0; i1 < os[2]; i1++)
                for (int i0 = 0; i0 < os[3]; i0++, oi++) {
                    const int64_t a_i = i3 * st0[0] + i2 * st0[1] + i1 * st0[2] + i0 * st0[3];
                    const int64_t b_i = i3 * st1[0] + i2 * st1[1] + i1 * st1[2] + i0 * st1[3];
                    switch (d->op) {
                    case ESPDL_ELT_ADD: /* esp-dl/dl/base/dl_base_add.cpp:8-44: exponents already equal */
                        store_sat(d->output, odt, oi, load_int(d->input0, idt, a_i) + load_int(d->input1, idt, b_i));
                        break;
                    case ESPDL_ELT_SUB: /* esp-dl/dl/base/dl_base_sub.cpp, same shape as add */
                        store_sat(d->output, odt, oi, load_int(d->input0, idt, a_i) - load_int(d->input1, idt, b_i));
                        break;
                    case ESPDL_ELT_MUL: { /* esp-dl/dl/base/dl_base_mul.cpp:9-46 */
                        int32_t t = (int32_t)(load_int(d->input0, idt, a_i) * load_int(d->input1, idt, b_i));
                        float out = (float)t * mul_scale;
                        store_sat(d->output, odt, oi, fround(out, mode));
                        break;
                    }
                    case ESPDL_ELT_REQUANTIZE: { /* esp-dl/dl/tensor/src/dl_tensor_base.cpp:223-404 */
                        if (idt == ESPDL_DTYPE_FLOAT) { /* :251-264 QuantizeLinear */
                            float x = ((const float *)d->input0)[a_i];
                            store_sat(d->output, odt, oi, quantize_f(x, dl_rescale(d->out_exponent), mode));
                        } else if (odt == ESPDL_DTYPE_FLOAT) { /* :283-298 DequantizeLinear */
                            ((float *)d->output)[oi] = (float)load_int(d->input0, idt, a_i) * dl_scale(d->in0_exponent);
                        } else if (d->in0_exponent == d->out_exponent) { /* :311-328 */
                            store_sat(d->output, odt, oi, load_int(d->input0, idt, a_i));
                        } else { /* :362-395 quantize(dequantize()) */
                            float src_scale = dl_scale(d->in0_exponent);
                            float inv_scale = (float)(1.0 / (double)dl_scale(d->out_exponent));
                            float tmp = (float)load_int(d->input0, idt, a_i) * src_scale;
                            store_sat(d->output, odt, oi, quantize_f(tmp, inv_scale, mode));
                        }
                        break;
                    }
                    case ESPDL_ELT_LUT: /* esp-dl/dl/base/dl_base_lut.cpp:10-15 (int8), :50-77 (int16) */
                        if (idt == ESPDL_DTYPE_INT16) {
                            const uint32_t value = (uint32_t)(uint16_t)((const int16_t *)d->input0)[a_i] ^ 0x8000u;
                            uint32_t index = value;
                            if (d->lut_shift > 0) {
                                index = value >> d->lut_shift;
                                const uint32_t rem = value & ((1u << d->lut_shift) - 1u), half = 1u << (d->lut_shift - 1);
                                if (mode == ESPDL_ROUND_HALF_EVEN ? (rem > half || (rem == half && (index & 1u))) : rem >= half)
                                    index++;
                            }
                            ((int16_t *)d->output)[oi] = ((const int16_t *)d->input1)[index];
                            break;
                        }
                        ((int8_t *)d->output)[oi] =
                            ((const int8_t *)d->input1)[(uint8_t)((const int8_t *)d->input0)[a_i] ^ 0x80u];
                        break;
                    case ESPDL_ELT_CLIP: { /* esp-dl/dl/module/include/dl_module_clip.hpp:78-90 */
                        int64_t v = clamp64(load_int(d->input0, idt, a_i), d->clip_lo, d->clip_hi);
                        store_sat(d->output, odt, oi, fround((float)v * clip_rescale, mode));
                        break;
                    }
                    case ESPDL_ELT_RELU: { /* esp-dl/dl/module/include/dl_module_relu.hpp:66-91 */
                        int64_t v = load_int(d->input0, idt, a_i);
                        if (d->in0_exponent == d->out_exponent) {
                            store_sat(d->output, odt, oi, v >= 0 ? v : 0);
                        } else {
                            float temp = (float)v * dl_scale(d->in0_exponent);
                            if (temp >= 0)
                                store_sat(d->output, odt, oi, fround(temp * dl_rescale(d->out_exponent), mode));
                            else
                                store_sat(d->output, odt, oi, 0);
                        }
                        break;
                    }
                    case ESPDL_ELT_PRELU: { /* esp-dl/dl/base/dl_base_prelu.cpp:5-19, shift esp-dl/dl/base/dl_base.hpp:2165-2168 */
                        int64_t v = load_int(d->input0, idt, a_i);
                        if (v < 0) {
                            int shift = d->out_exponent - d->in0_exponent - d->in1_exponent;
                            int64_t prod = v * load_int(d->input1, idt, i0 % C);
                            if (idt == ESPDL_DTYPE_INT8)
                                prod = (int32_t)prod;
                            /* DL_RIGHT_SHIFT: plain arithmetic shift, no rounding */
                            v = shift > 0 ? (prod >> shift) : (int64_t)((uint64_t)prod << (-shift));
                            if (idt == ESPDL_DTYPE_INT8)
                                v = (int32_t)v;
                        }
                        store_sat(d->output, odt, oi, v);
                        break;
                    }
                    case ESPDL_ELT_MAX:   /* esp-dl/dl/base/dl_base_max.cpp:9-50: raw integers, exponents not looked at */
                    case ESPDL_ELT_MIN: { /* esp-dl/dl/base/dl_base_min.cpp */
                        const int64_t a = load_int(d->input0, idt, a_i), b = load_int(d->input1, idt, b_i);
                        store_sat(d->output, odt, oi, d->op == ESPDL_ELT_MAX ? (a > b ? a : b) : (a < b ? a : b));
                        break;
                    }
                    case ESPDL_ELT_DIV: { /* esp-dl/dl/base/dl_base_div.cpp:87-207 */
                        const int64_t a = load_int(d->input0, idt, a_i), b = load_int(d->input1, idt, b_i);
                        const int64_t hi = idt == ESPDL_DTYPE_INT8 ? INT8_MAX : INT16_MAX, lo = -hi - 1;
                        if (div_table0) {
                            const float a_f = (float)a * div_scale;
                            store_sat(d->output, odt, oi, b == 0 ? (a_f > 0 ? hi : lo) : fround(a_f / (float)b, mode));
                        } else if (a == 0) {
                            store_sat(d->output, odt, oi, 0);
                        } else if (b == 0) {
                            store_sat(d->output, odt, oi, a > 0 ? hi : lo);
                        } else if (div_n1) {
                            const float rescale = div_scale / (float)b;
                            store_sat(d->output, odt, oi, fround((float)a * rescale, mode));
                        } else {
                            const float scaled = (float)a * div_scale;
                            store_sat(d->output, odt, oi, fround(scaled / (float)b, mode));
                        }
                        break;
                    }
                    case ESPDL_ELT_MOD: { /* esp-dl/dl/base/dl_base_mod.cpp:9-62 */
                        const float a_val = (float)load_int(d->input0, idt, a_i) * dl_scale(d->in0_exponent);
                        const float b_val = (float)load_int(d->input1, idt, b_i) * dl_scale(d->in1_exponent);
                        const float r = b_val != 0.0f ? fmodf(a_val, b_val) : 0.0f;
                        store_sat(d->output, odt, oi, fround(r * dl_rescale(d->out_exponent), mode));
                        break;
                    }
                    case ESPDL_ELT_POW: { /* esp-dl/dl/base/dl_base_pow.cpp:9-63 (the three loops differ only in what is hoisted) */
                        const float base_val = (float)load_int(d->input0, idt, a_i) * dl_scale(d->in0_exponent);
                        const float exp_val = (float)load_int(d->input1, idt, b_i) * dl_scale(d->in1_exponent);
                        const float r = powf(base_val, exp_val) * dl_rescale(d->out_exponent);
                        /* (int)floorf(r + 0.5) of a NaN, an infinity or a value past int32 is INT32_MIN on x86 (cvttss2si);
                         * written out so that the restatement does not rest on undefined behaviour */
                        store_sat(d->output, odt, oi, !(fabsf(r) < 2147483520.f) ? INT32_MIN : fround(r, mode));
                        break;
                    }
                    case ESPDL_ELT_GREATER: /* esp-dl/dl/base/dl_base_greater.cpp:9-44 and its siblings: raw integers */
                    case ESPDL_ELT_GREATER_EQUAL:
                    case ESPDL_ELT_EQUAL:
                    case ESPDL_ELT_LESS:
                    case ESPDL_ELT_LESS_EQUAL: {
                        const int64_t a = load_int(d->input0, idt, a_i), b = load_int(d->input1, idt, b_i);
                        const int r = d->op == ESPDL_ELT_GREATER ? a > b : d->op == ESPDL_ELT_GREATER_EQUAL ? a >= b :
                            d->op == ESPDL_ELT_EQUAL ? a == b : d->op == ESPDL_ELT_LESS ? a < b : a <= b;
                        ((uint8_t *)d->output)[oi] = (uint8_t)r;
                        break;
                    }
                    default:
                        return ESPDL_ERR_UNSUPPORTED;
                    }
                }
    return ESPDL_OK;
}

/* ------------------------------------------------------------- pooling */
/* Max: esp-dl/dl/base/dl_base_max_pool2d.cpp:9-27 over in-bounds taps only (shell
 * esp-dl/dl/base/dl_base_pool2d.hpp shrinks the window at borders).
 * Avg / global avg: esp-dl/dl/base/dl_base_avg_pool2d.cpp:10-55: integer sum of the in-bounds
 * taps, then sat(round((float)sum * scale)), scale = (2^e_in * (1.f/area)) * 2^-e_out with
 * area = kh*kw of the full window (esp-dl/dl/base/dl_base_pool2d.hpp:132). */
int oracle_pool(const espdl_pool_desc *d)
{
    if (!d || !d->input || !d->output)
        return ESPDL_ERR_INVALID_ARG;
    const int is16 = d->dtype == ESPDL_DTYPE_INT16;
    int kh = d->kh, kw = d->kw, sh = d->stride_h, sw = d->stride_w, oh = d->out_h, ow = d->out_w;
    int pt = d->pad_top, pl = d->pad_left;
    if (d->op == ESPDL_POOL_GLOBAL_AVG) {
        kh = d->in_h, kw = d->in_w, sh = sw = 1, oh = ow = 1, pt = pl = 0;
    }
    const float inv_area = 1.f / (float)(kh * kw);
    const float scale = dl_scale(d->in_exponent) * inv_area * dl_rescale(d->out_exponent);
    for (int n = 0; n < d->n; n++)
        for (int oy = 0; oy < oh; oy++)
            for (int ox = 0; ox < ow; ox++)
                for (int c = 0; c < d->c; c++) {
                    int64_t sum = 0, mx = INT64_MIN;
                    for (int ky = 0; ky < kh; ky++) {
                        int iy = oy * sh + ky - pt;
                        if (iy < 0 || iy >= d->in_h)
                            continue;
                        for (int kx = 0; kx < kw; kx++) {
                            int ix = ox * sw + kx - pl;
                            if (ix < 0 || ix >= d->in_w)
                                continue;
                            int64_t v = load_int(d->input, d->dtype, (((int64_t)n * d->in_h + iy) * d->in_w + ix) * d->c + c);
                            sum += v;
                            if (v > mx)
                                mx = v;
                        }
                    }
                    int64_t oi = (((int64_t)n * oh + oy) * ow + ox) * d->c + c;
                    if (d->op == ESPDL_POOL_MAX)
                        store_sat(d->output, d->dtype, oi, mx);
                    else
                        store_sat(d->output, d->dtype, oi, fround_half_up((float)(is16 ? sum : (int32_t)sum) * scale));
                }
    return ESPDL_OK;
}

/* -------------------------------------------------------------- resize */
/* esp-dl/dl/base/dl_base_resize.cpp:7-35 (value), :239-268 (coordinates),
 * esp-dl/dl/base/dl_base_resize.hpp:80-85 (scale/shift).  The value is a plain cast
 * of round(), without saturation. */
/* linear_coeffs + resize_linear_c1: esp-dl/dl/base/dl_base_resize.cpp:80-236 */
static void oracle_linear_coeffs(int out_x, int *in_x, float *r0, float *r1, int in_length, float scale_inv, int align)
{
    float fx = align ? out_x * scale_inv : (out_x + 0.5f) * scale_inv - 0.5f;
    *in_x = (int)floorf(fx);
    fx -= *in_x;
    if (*in_x < 0) {
        *in_x = 0;
        fx = 0.f;
    }
    if (*in_x >= in_length - 1) {
        *in_x = in_length - 2;
        fx = 1.f;
    }
    *r0 = 1.f - fx;
    *r1 = fx;
}

static int oracle_resize_linear(const espdl_resize_desc *d)
{
    const int align = d->mode == 2, one_d = d->in_h == 1 && d->out_h == 1;
    if (d->in_w < 2 || (!one_d && d->in_h < 2))
        return ESPDL_ERR_UNSUPPORTED;
    float sh = d->scale_h, sw = d->scale_w;
    if (align) {
        sh = one_d ? 1.f : (d->out_h - 1) / (float)(d->in_h - 1);
        sw = (d->out_w - 1) / (float)(d->in_w - 1);
    }
    const float sh_inv = 1 / sh, sw_inv = 1 / sw;
    const float in_scale = dl_scale(d->in_exponent), out_rescale = dl_rescale(d->out_exponent);
    const int ops = d->out_pixel_stride ? d->out_pixel_stride : d->c;
    const int8_t *in = (const int8_t *)d->input;
    for (int n = 0; n < d->n; n++)
        for (int y = 0; y < d->out_h; y++) {
            int iy = 0;
            float yr0 = 1.f, yr1 = 0.f;
            if (!one_d)
                oracle_linear_coeffs(y, &iy, &yr0, &yr1, d->in_h, sh_inv, align);
            for (int x = 0; x < d->out_w; x++) {
                int ix;
                float xr0, xr1;
                oracle_linear_coeffs(x, &ix, &xr0, &xr1, d->in_w, sw_inv, align);
                for (int c = 0; c < d->c; c++) {
                    const int8_t *row0 = in + (((int64_t)n * d->in_h + iy) * d->in_w + ix) * d->c + c;
                    float v = (float)row0[0] * in_scale * xr0 + (float)row0[d->c] * in_scale * xr1;
                    if (!one_d) {
                        const int8_t *row1 = row0 + (int64_t)d->in_w * d->c;
                        const float w = (float)row1[0] * in_scale * xr0 + (float)row1[d->c] * in_scale * xr1;
                        v = v * yr0 + w * yr1;
                    }
                    int q = fround_half_up(v * out_rescale);
                    q = q < -128 ? -128 : (q > 127 ? 127 : q);
                    ((int8_t *)d->output)[(((int64_t)n * d->out_h + y) * d->out_w + x) * ops + c] = (int8_t)q;
                }
            }
        }
    return ESPDL_OK;
}

int oracle_resize(const espdl_resize_desc *d)
{
    if (!d || !d->input || !d->output)
        return ESPDL_ERR_INVALID_ARG;
    if (d->dtype != ESPDL_DTYPE_INT8) /* resize<int16_t> is an empty function: esp-dl/dl/base/dl_base_resize.cpp:298-309 */
        return ESPDL_ERR_UNSUPPORTED;
    if (d->mode != 0)
        return oracle_resize_linear(d);
    int shift = d->out_exponent - d->in_exponent, oscale = 1;
    if (shift < 0) {
        oscale = 1 << (-shift);
        shift = 0;
    }
    const float sh_inv = 1 / d->scale_h, sw_inv = 1 / d->scale_w;
    const int ops = d->out_pixel_stride ? d->out_pixel_stride : d->c;
    const int two = d->scale_h == 2 && d->scale_w == 2;
    for (int n = 0; n < d->n; n++)
        for (int y = 0; y < d->out_h; y++) {
            int iy = two ? y / 2 : (int)(y * sh_inv);
            if (iy > d->in_h - 1)
                iy = d->in_h - 1;
            for (int x = 0; x < d->out_w; x++) {
                int ix = two ? x / 2 : (int)(x * sw_inv);
                if (ix > d->in_w - 1)
                    ix = d->in_w - 1;
                for (int c = 0; c < d->c; c++) {
                    int64_t ii = (((int64_t)n * d->in_h + iy) * d->in_w + ix) * d->c + c;
                    int64_t oi = (((int64_t)n * d->out_h + y) * d->out_w + x) * ops + c;
                    int v = fround_half_up((float)load_int(d->input, d->dtype, ii) * (float)oscale / (float)(1 << shift));
                    if (d->dtype == ESPDL_DTYPE_INT8)
                        ((int8_t *)d->output)[oi] = (int8_t)v;
                    else
                        ((int16_t *)d->output)[oi] = (int16_t)v;
                }
            }
        }
    return ESPDL_OK;
}

/* ---------------------------------------------------------------- copy */
int oracle_copy(const espdl_copy_desc *d)
{
    if (!d || !d->src || !d->dst || d->ndim < 1 || d->ndim > 6)
        return ESPDL_ERR_INVALID_ARG;
    int shp[6] = {1, 1, 1, 1, 1, 1};
    int64_t ss[6] = {0}, ds[6] = {0};
    for (int i = 0; i < d->ndim; i++) {
        shp[6 - d->ndim + i] = d->shape[i];
        ss[6 - d->ndim + i] = d->src_stride[i];
        ds[6 - d->ndim + i] = d->dst_stride[i];
    }
    const int es = d->elem_size;
    for (int a = 0; a < shp[0]; a++)
        for (int b = 0; b < shp[1]; b++)
            for (int c = 0; c < shp[2]; c++)
                for (int e = 0; e < shp[3]; e++)
                    for (int f = 0; f < shp[4]; f++)
                        for (int g = 0; g < shp[5]; g++) {
                            int64_t si = a * ss[0] + b * ss[1] + c * ss[2] + e * ss[3] + f * ss[4] + g * ss[5];
                            int64_t di = a * ds[0] + b * ds[1] + c * ds[2] + e * ds[3] + f * ds[4] + g * ds[5];
                            memcpy((char *)d->dst + di * es, (const char *)d->src + si * es, (size_t)es);
                        }
    return ESPDL_OK;
}

/* ------------------------------------------------------------- softmax */
/* esp-dl/dl/module/include/dl_module_softmax.hpp:148-187: y_i = T[x_i+128] / sum_j T[x_j+128],
 * sequential fp32 sum in index order; T from dl::tool::gen_lut_8bit
 * (esp-dl/dl/tool/src/dl_tool.cpp:258-268).  A following QuantizeLinear
 * (esp-dl/dl/tensor/src/dl_tensor_base.cpp:251-264) is folded in when out_dtype is an integer type. */
void oracle_softmax_table(float *table, int in_exponent)
{
    float scale = dl_scale(in_exponent);
    for (int i = 0; i < 256; i++) table[i] = expf(scale * (float)(i - 128));
}

int oracle_softmax(const espdl_softmax_desc *d)
{
    if (!d || !d->input || !d->output || !d->exp_table)
        return ESPDL_ERR_INVALID_ARG;
    const float inv_scale = dl_rescale(d->out_exponent);
    const int inner = d->inner > 1 ? d->inner : 1;
    const float scale = dl_scale(d->in_exponent);
    for (int r = 0; r < d->rows; r++) {
        /* a row: len elements that lie `inner` apart (any axis, dl_module_log_softmax.hpp:185-215) */
        const int64_t base = (int64_t)(r / inner) * d->len * inner + r % inner;
        const int8_t *x = d->input + base;
        float sum = 0.f;
        for (int i = 0; i < d->len; i++) sum += d->exp_table[x[(int64_t)i * inner] + 128];
        const float log_sum = d->log ? logf(sum) : 0.f; /* esp-dl/dl/module/include/dl_module_log_softmax.hpp:168-175 */
        for (int i = 0; i < d->len; i++) {
            const int xi = x[(int64_t)i * inner];
            float y = d->log ? scale * xi - log_sum : d->exp_table[xi + 128] / sum;
            int64_t oi = base + (int64_t)i * inner;
            if (d->out_dtype == ESPDL_DTYPE_FLOAT)
                ((float *)d->output)[oi] = y;
            else
                store_sat(d->output, d->out_dtype, oi, fround(y * inv_scale, d->round_mode));
        }
    }
    return ESPDL_OK;
}

/* ---------------------------------------------------------------- image pre-processing */
/* Table of NormQuant (esp-dl/vision/image/dl_image_norm_quant.hpp:13-31): entry [c][v] =
 * quantize((v - mean[c]) * (1/std[c]), inv_scale), quantize = clip(round(x * inv_scale))
 * (esp-dl/dl/tensor/src/dl_tensor_base.cpp:18-30), inv_scale = 2^-exponent.  `table` holds channels*256 entries
 * of int8 (bits 8) or int16 (bits 16). */
void oracle_norm_quant_table(void *table, int channels, const float *mean, const float *std, int exponent, int bits, int round_mode)
{
    const float inv_scale = exponent > 0 ? 1.f / (float)(1 << exponent) : (float)(1 << -exponent);
    for (int c = 0; c < channels; c++) {
        const float inv_std = 1.f / std[c];
        for (int j = 0; j < 256; j++) {
            const float x = ((float)j - mean[c]) * inv_std;
            int q = fround(x * inv_scale, round_mode);
            if (bits == 8) {
                q = q < -128 ? -128 : (q > 127 ? 127 : q);
                ((int8_t *)table)[c * 256 + j] = (int8_t)q;
            } else {
                q = q < -32768 ? -32768 : (q > 32767 ? 32767 : q);
                ((int16_t *)table)[c * 256 + j] = (int16_t)q;
            }
        }
    }
}

/* ImagePreprocessor::preprocess with the nearest-neighbour maps of ImageTransformer::gen_xy_map
 * (esp-dl/vision/image/dl_image_process.cpp:488-536), the letterbox border (dl_image_preprocessor.cpp:108-131,
 * background converted like a pixel: dl_image_process.cpp:438-474) and RGB8882RGB888
 * (dl_image_color_rgb8882rgb888.hpp:51-63).  Host pointers. */
int oracle_image_preprocess(const espdl_image_desc *d)
{
    if (!d || !d->input || !d->output || !d->lut || (d->channels != 1 && d->channels != 3))
        return ESPDL_ERR_INVALID_ARG;
    const int whole = d->crop_x0 == 0 && d->crop_y0 == 0 && d->crop_x1 == 0 && d->crop_y1 == 0;
    const int x0 = whole ? 0 : d->crop_x0, y0 = whole ? 0 : d->crop_y0, x1 = whole ? d->src_w : d->crop_x1, y1 = whole ? d->src_h : d->crop_y1;
    const int inner_w = d->dst_w - d->border_left - d->border_right, inner_h = d->dst_h - d->border_top - d->border_bottom;
    const int src_w = x1 - x0, src_h = y1 - y0;
    const int same = src_w == inner_w && src_h == inner_h;
    const float isx = (float)src_w / (float)inner_w, isy = (float)src_h / (float)inner_h;
    const int ch = d->channels, is8 = d->out_dtype == ESPDL_DTYPE_INT8;
    for (int n = 0; n < d->n; n++)
        for (int y = 0; y < d->dst_h; y++)
            for (int x = 0; x < d->dst_w; x++) {
                const int xi = x - d->border_left, yi = y - d->border_top;
                uint8_t v[3] = {0, 0, 0};
                if (xi < 0 || xi >= inner_w || yi < 0 || yi >= inner_h) {
                    for (int c = 0; c < ch; c++) v[c] = d->bg[c];
                } else {
                    int sx = same ? xi + x0 : (int)((float)xi * isx) + x0;
                    int sy = same ? yi + y0 : (int)((float)yi * isy) + y0;
                    if (!same) {
                        sx = sx < x1 - 1 ? sx : x1 - 1;
                        sy = sy < y1 - 1 ? sy : y1 - 1;
                    }
                    const uint8_t *src = d->input + (((int64_t)n * d->src_h + sy) * d->src_w + sx) * ch;
                    for (int c = 0; c < ch; c++) v[c] = src[c];
                }
                const int64_t o = (((int64_t)n * d->dst_h + y) * d->dst_w + x) * ch;
                for (int c = 0; c < ch; c++) {
                    const int sc = (ch == 3 && d->swap_rb) ? 2 - c : c;
                    if (is8)
                        ((int8_t *)d->output)[o + c] = ((const int8_t *)d->lut)[c * 256 + v[sc]];
                    else
                        ((int16_t *)d->output)[o + c] = ((const int16_t *)d->lut)[c * 256 + v[sc]];
                }
            }
    return ESPDL_OK;
}

/* ---------------------------------------------------------------- detection post-processing (one image) */
/* dl::detect::yolo11PostProcessor::parse_stage + DetectPostprocessor::nms + get_result
 * (esp-dl/vision/detect/dl_detect_yolo11_postprocessor.cpp:8-73, dl_detect_postprocessor.cpp:5-50) with the helpers of
 * esp-dl/dl/math/include/dl_math.hpp:200-258.  Candidates are kept in a list sorted by descending score, a new one
 * goes behind those of equal score (std::upper_bound with greater_box). */
typedef struct oracle_det_stage {
    const int8_t *score; /* [h][w][classes] */
    const int8_t *box;   /* [h][w][64] */
    int h, w, classes;
    int score_exponent, box_exponent;
    int stride_y, stride_x, offset_y, offset_x;
} oracle_det_stage;

typedef struct { int category; float score; int box[4]; } det_t;

static float det_sigmoid(float x) { return 1.0 / (1.0 + expf(-x)); }
static float det_inverse_sigmoid(float x) { return -logf(1.0 / x - 1); }
static float det_dfl_integral(float *data, int reg_max)
{
    float max_input = data[0];
    for (int i = 1; i <= reg_max; i++) max_input = max_input > data[i] ? max_input : data[i];
    float sum = 0;
    for (int i = 0; i <= reg_max; i++) {
        data[i] = expf(data[i] - max_input);
        sum += data[i];
    }
    for (int i = 0; i <= reg_max; i++) data[i] /= sum;
    float acc = 0;
    for (int i = 0; i <= reg_max; i++) acc += data[i] * i;
    return acc;
}

int oracle_yolo11_postprocess(const oracle_det_stage *stages, int n_stages, float score_thr, float nms_thr, int top_k, float inv_scale_x,
                              float inv_scale_y, int border_left, int border_top, int width, int height, int round_mode, int max_results,
                              int *boxes, float *scores)
{
    int cap = 1024, n = 0;
    det_t *list = (det_t *)malloc(sizeof(det_t) * cap);
    for (int s = 0; s < n_stages; s++) {
        const oracle_det_stage *st = &stages[s];
        const float score_exp = dl_scale(st->score_exponent), box_exp = dl_scale(st->box_exponent);
        int thr = fround(det_inverse_sigmoid(score_thr) * (1.f / score_exp), round_mode);
        thr = thr < -128 ? -128 : (thr > 127 ? 127 : thr);
        const int8_t *sp = st->score, *bp = st->box;
        for (int y = 0; y < st->h; y++)
            for (int x = 0; x < st->w; x++, bp += 64)
                for (int c = 0; c < st->classes; c++, sp++) {
                    if (*sp <= (int8_t)thr)
                        continue;
                    const int center_y = y * st->stride_y + st->offset_y, center_x = x * st->stride_x + st->offset_x;
                    float d[64];
                    for (int i = 0; i < 64; i++) d[i] = (float)bp[i] * box_exp;
                    det_t nb;
                    nb.category = c;
                    nb.score = det_sigmoid((float)*sp * score_exp);
                    nb.box[0] = (int)(((center_x - det_dfl_integral(d, 15) * st->stride_x) - border_left) * inv_scale_x);
                    nb.box[1] = (int)(((center_y - det_dfl_integral(d + 16, 15) * st->stride_y) - border_top) * inv_scale_y);
                    nb.box[2] = (int)(((center_x + det_dfl_integral(d + 32, 15) * st->stride_x) - border_left) * inv_scale_x);
                    nb.box[3] = (int)(((center_y + det_dfl_integral(d + 48, 15) * st->stride_y) - border_top) * inv_scale_y);
                    int pos = 0; /* first element with a strictly lower score */
                    while (pos < n && !(nb.score > list[pos].score)) pos++;
                    if (n == cap) {
                        cap *= 2;
                        list = (det_t *)realloc(list, sizeof(det_t) * cap);
                    }
                    memmove(list + pos + 1, list + pos, sizeof(det_t) * (size_t)(n - pos));
                    list[pos] = nb;
                    n++;
                }
    }
    /* nms */
    char *dead = (char *)calloc((size_t)n + 1, 1);
    int kept_number = 0, end = n;
    for (int k = 0; k < end; k++) {
        if (dead[k])
            continue;
        kept_number++;
        if (kept_number >= top_k) {
            end = k + 1;
            break;
        }
        const int kept_area = (list[k].box[2] - list[k].box[0] + 1) * (list[k].box[3] - list[k].box[1] + 1);
        for (int o = k + 1; o < end; o++) {
            if (dead[o])
                continue;
            const int lx = list[k].box[0] > list[o].box[0] ? list[k].box[0] : list[o].box[0];
            const int ly = list[k].box[1] > list[o].box[1] ? list[k].box[1] : list[o].box[1];
            const int rx = list[k].box[2] < list[o].box[2] ? list[k].box[2] : list[o].box[2];
            const int ry = list[k].box[3] < list[o].box[3] ? list[k].box[3] : list[o].box[3];
            const int ih = ry - ly + 1, iw = rx - lx + 1;
            if (ih > 0 && iw > 0) {
                const int other_area = (list[o].box[2] - list[o].box[0] + 1) * (list[o].box[3] - list[o].box[1] + 1);
                const int inter = ih * iw;
                const float iou = (float)inter / (kept_area + other_area - inter);
                if (iou > nms_thr)
                    dead[o] = 1;
            }
        }
    }
    int out = 0;
    for (int k = 0; k < end && out < max_results; k++) {
        if (dead[k])
            continue;
        boxes[5 * out] = list[k].category;
        for (int j = 0; j < 4; j++) {
            const int lim = (j % 2 == 0 ? width : height) - 1;
            const int v = list[k].box[j];
            boxes[5 * out + 1 + j] = v < 0 ? 0 : (v > lim ? lim : v);
        }
        scores[out++] = list[k].score;
    }
    free(dead);
    free(list);
    return out;
}

/* ---------------------------------------------------------------- reductions */
/* ReduceBase::forward_template with ReduceMean / ReduceSum / ReduceMax / ReduceMin::reduce
 * (esp-dl/dl/module/include/dl_module_reduce_base.hpp:121-262, dl_module_reduce_mean.hpp:17-45,
 * dl_module_reduce_sum.hpp:17-42, dl_module_reduce_max.hpp:12-37, dl_module_reduce_min.hpp:13-38). */
int oracle_reduce(const espdl_reduce_desc *d)
{
    if (!d || !d->input || !d->output || d->ndim < 1 || d->ndim > 6)
        return ESPDL_ERR_INVALID_ARG;
    const int is8 = d->dtype == ESPDL_DTYPE_INT8;
    int64_t strides[6], total = 1, count = 1;
    for (int i = d->ndim - 1; i >= 0; i--) {
        strides[i] = total;
        total *= d->shape[i];
    }
    for (int i = 0; i < d->ndim; i++)
        if (d->reduce[i])
            count *= d->shape[i];
    const int64_t outputs = total / count;
    const int64_t lo = is8 ? -128 : -32768, hi = is8 ? 127 : 32767;
    for (int64_t o = 0; o < outputs; o++) {
        int64_t base = 0, rem = o;
        for (int i = d->ndim - 1; i >= 0; i--)
            if (!d->reduce[i]) {
                base += (rem % d->shape[i]) * strides[i];
                rem /= d->shape[i];
            }
        int64_t acc = d->op == ESPDL_REDUCE_MAX ? lo : (d->op == ESPDL_REDUCE_MIN ? hi : 0);
        float facc = d->op == ESPDL_REDUCE_PROD ? 1.f : 0.f; /* V_T = float: int8 product, sums of exponentials */
        double dacc = 1.0;                                    /* V_T = double: int16 product */
        for (int64_t r = 0; r < count; r++) {
            int64_t off = base, rr = r;
            for (int i = d->ndim - 1; i >= 0; i--)
                if (d->reduce[i]) {
                    off += (rr % d->shape[i]) * strides[i];
                    rr /= d->shape[i];
                }
            const int64_t v = load_int(d->input, d->dtype, off);
            if (d->op == ESPDL_REDUCE_PROD) {
                /* ReduceBase::reduce with an exponent, dl_module_reduce_base.hpp:100-118: float tmp = x * input_scale;
                 * sum = sum * tmp in V_T (dl_module_reduce_prod.hpp:18-21, 54-60) */
                const float tmp = (float)v * dl_scale(d->in_exponent);
                if (is8)
                    facc = facc * tmp;
                else
                    dacc = dacc * tmp;
            } else if (d->op == ESPDL_REDUCE_LOG_SUM_EXP) {
                /* dl_module_reduce_log_sum_exp.hpp:27-44: int8 adds exp_table[x + 128] (tool::gen_lut_8bit(expf)), int16 adds
                 * expf(x * input_scale); V_T = float for both (:112-123) */
                if (is8)
                    facc = facc + expf(dl_scale(d->in_exponent) * (float)((int)v + 128 - 128));
                else
                    facc = facc + expf((float)v * dl_scale(d->in_exponent));
            } else if (d->op == ESPDL_REDUCE_MAX)
                acc = acc > v ? acc : v;
            else if (d->op == ESPDL_REDUCE_MIN)
                acc = acc < v ? acc : v;
            else if (d->op == ESPDL_REDUCE_L1) /* esp-dl/dl/module/include/dl_module_reduce_l1.hpp:18-21 */
                acc += v < 0 ? -v : v;
            else if (d->op == ESPDL_REDUCE_SUM_SQUARE || d->op == ESPDL_REDUCE_L2) /* dl_module_reduce_base.hpp:77-80 */
                acc += v * v;
            else
                acc += v;
        }
        if (is8)
            acc = (int32_t)acc; /* the int8 accumulator is an int32_t */
        int64_t q = acc;
        if (d->op == ESPDL_REDUCE_MEAN) {
            /* tool::round(tmp * input_scale / count * output_scale): the sum is an int32 (int8) or int64 (int16) */
            float f = is8 ? (float)(int32_t)acc : (float)acc;
            f = f * dl_scale(d->in_exponent);
            f = f / (float)(size_t)count;
            f = f * dl_rescale(d->out_exponent);
            q = fround(f, d->round_mode);
        } else if (d->op == ESPDL_REDUCE_PROD) { /* dl_module_reduce_prod.hpp:39-47 */
            if (is8) {
                q = fround(facc * dl_rescale(d->out_exponent), d->round_mode);
            } else {
                const double t = dacc * dl_rescale(d->out_exponent); /* tool::round(double), dl_tool.cpp:51-80 */
                q = d->round_mode == ESPDL_ROUND_HALF_EVEN ? (int)rint(t) : (int)floor(t + 0.5);
            }
        } else if (d->op == ESPDL_REDUCE_LOG_SUM) { /* dl_module_reduce_log_sum.hpp:36-45 */
            const float tmp = is8 ? (float)((int32_t)acc * dl_scale(d->in_exponent)) : (float)(acc * dl_scale(d->in_exponent));
            q = fround(logf(tmp) * dl_rescale(d->out_exponent), d->round_mode);
        } else if (d->op == ESPDL_REDUCE_LOG_SUM_EXP) { /* dl_module_reduce_log_sum_exp.hpp:62-68, 98-103 */
            q = fround(logf(facc) * dl_rescale(d->out_exponent), d->round_mode);
        } else if (d->op == ESPDL_REDUCE_SUM || d->op == ESPDL_REDUCE_L1) {
            q = shift_and_round(acc, d->out_exponent - d->in_exponent, d->round_mode, is8 ? 32 : 64);
        } else if (d->op == ESPDL_REDUCE_SUM_SQUARE) { /* esp-dl/dl/module/include/dl_module_reduce_sum_square.hpp:36-39 */
            q = shift_and_round(acc, d->out_exponent - 2 * d->in_exponent, d->round_mode, is8 ? 32 : 64);
        } else if (d->op == ESPDL_REDUCE_L2) {
            /* esp-dl/dl/module/include/dl_module_reduce_l2.hpp:37-42 with math::sqrt_newton, esp-dl/dl/math/include/
             * dl_math.hpp:83-97 (the iteration is capped at 100 steps here; it ends by itself long before) */
            const float x = (is8 ? (float)(int32_t)acc : (float)acc) * dl_scale(2 * d->in_exponent);
            float r = x;
            if (x != 0.f) {
                for (int it = 0; it < 100; it++) {
                    const float last = r;
                    r = (float)((last + x / last) * 0.5);
                    if (!(fabsf(r - last) > 0.00001f))
                        break;
                }
            }
            q = fround(r * dl_rescale(d->out_exponent), d->round_mode);
        }
        store_sat(d->output, d->dtype, o, q);
    }
    return ESPDL_OK;
}

/* ---------------------------------------------------------------- Pad */
/* TensorBase::pad / base::padND (esp-dl/dl/base/dl_base_pad.cpp:18-66 per axis): constant, edge, reflect. */
int oracle_pad(const espdl_pad_desc *d)
{
    if (!d || !d->input || !d->output || d->ndim < 1 || d->ndim > 6)
        return ESPDL_ERR_INVALID_ARG;
    int64_t istride[6], oshape[6], total = 1, stride = 1;
    for (int i = d->ndim - 1; i >= 0; i--) {
        istride[i] = stride;
        stride *= d->shape[i];
        oshape[i] = d->shape[i] + d->pad_begin[i] + d->pad_end[i];
        total *= oshape[i];
    }
    for (int64_t o = 0; o < total; o++) {
        int64_t rem = o, off = 0;
        int inside = 1;
        for (int k = d->ndim - 1; k >= 0; k--) {
            int64_t i = rem % oshape[k] - d->pad_begin[k];
            rem /= oshape[k];
            const int64_t n = d->shape[k];
            if (i < 0 || i >= n) {
                if (d->mode == ESPDL_PAD_CONSTANT)
                    inside = 0;
                else if (d->mode == ESPDL_PAD_EDGE)
                    i = i < 0 ? 0 : n - 1;
                else
                    i = i < 0 ? -i : 2 * (n - 1) - i;
                if (i < 0) i = 0;
                if (i > n - 1) i = n - 1;
            }
            off += i * istride[k];
        }
        if (inside)
            memcpy((char *)d->output + o * d->elem_size, (const char *)d->input + off * d->elem_size, (size_t)d->elem_size);
        else
            memcpy((char *)d->output + o * d->elem_size, &d->constant, (size_t)d->elem_size); /* little endian */
    }
    return ESPDL_OK;
}

int oracle_num_threads(void)
{
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ---------------------------------------------------------------- Gather, SpaceToDepth, DepthToSpace */
/* dl::module::Gather::forward_template (esp-dl/dl/module/include/dl_module_gather.hpp:66-77). */
int oracle_gather(const espdl_gather_desc *d)
{
    if (!d || !d->input || !d->output || !d->indices)
        return ESPDL_ERR_INVALID_ARG;
    const size_t row = (size_t)d->inner * d->elem_size;
    for (int64_t o = 0; o < d->outer; o++)
        for (int i = 0; i < d->num_indices; i++) {
            const int idx = d->indices[i];
            if (idx < 0 || idx >= d->axis_size)
                continue;
            memcpy((char *)d->output + (size_t)(o * d->num_indices + i) * row, (const char *)d->input + (size_t)(o * d->axis_size + idx) * row, row);
        }
    return ESPDL_OK;
}

/* mode 0: SpaceToDepth (esp-dl/dl/module/include/dl_module_space_to_depth.hpp:20-47); mode 1 / 2: DepthToSpace "DCR" /
 * "CRD" (esp-dl/dl/module/include/dl_module_depth_to_space.hpp:20-72).  NHWC, h / w / c are the INPUT extents.  The
 * reference's DCR index rule (out_c = c % blocksize, row = c / blocksize^2) addresses the output consistently only
 * when the output has `blocksize` channels; other shapes are rejected here. */
int oracle_depth_space(const void *input, void *output, int elem_size, int n, int h, int w, int c, int bs, int mode)
{
    if (!input || !output || bs < 1)
        return ESPDL_ERR_INVALID_ARG;
    const int b2 = bs * bs;
    if (mode == 0 ? (h % bs || w % bs) : (c % b2))
        return ESPDL_ERR_INVALID_ARG;
    if (mode == 1 && c / b2 != bs)
        return ESPDL_ERR_UNSUPPORTED;
    const char *in = (const char *)input;
    for (int b = 0; b < n; b++)
        for (int y = 0; y < h; y++)
            for (int x = 0; x < w; x++)
                for (int ch = 0; ch < c; ch++, in += elem_size) {
                    int64_t idx;
                    if (mode == 0) {
                        const int oc = c * b2, out_c = ch * b2 + (y % bs) * bs + x % bs;
                        idx = (int64_t)b * h * w * c + (int64_t)(y / bs) * (w / bs) * oc + (int64_t)(x / bs) * oc + out_c;
                    } else {
                        const int oc = c / b2;
                        const int64_t h_offset = (int64_t)w * bs * oc;
                        int out_c, oy, ox;
                        if (mode == 2) {
                            out_c = ch / b2, oy = y * bs + (ch % b2) / bs, ox = x * bs + ch % bs;
                        } else {
                            out_c = ch % bs, oy = y * bs + ch / b2, ox = x * bs + (ch % b2) / bs;
                        }
                        idx = (int64_t)b * h * w * c + oy * h_offset + (int64_t)ox * oc + out_c;
                    }
                    memcpy((char *)output + idx * elem_size, in, elem_size);
                }
    return ESPDL_OK;
}

/* ---------------------------------------------------------------- RMSNormalization / LayerNormalization */
/* math::sqrt_newton, esp-dl/dl/math/include/dl_math.hpp:83-97 (capped at 100 steps; it ends by itself long before) */
static float oracle_sqrt_newton(float x)
{
    if (x == 0.f)
        return 0.f;
    float r = x;
    for (int it = 0; it < 100; it++) {
        const float last = r;
        r = (float)((last + x / last) * 0.5);
        if (!(fabsf(r - last) > 0.00001f))
            break;
    }
    return r;
}

int oracle_norm(const espdl_norm_desc *d)
{
    if (!d || !d->input || !d->output || d->len <= 0)
        return ESPDL_ERR_INVALID_ARG;
    const int is8 = d->dtype == ESPDL_DTYPE_INT8, mode = d->round_mode;
    const float input_scale = dl_scale(d->in_exponent), output_scale = dl_rescale(d->out_exponent);
    if (d->op == ESPDL_NORM_LP) {
        /* dl::module::LpNormalization::forward_int8 / forward_int16 with compute_quant_inv_norm(_strided)
         * (esp-dl/dl/module/include/dl_module_lp_normalization.hpp:122-262, 328-356); math::fast_inv_sqrt is
         * 1.0f / sqrtf(x) because DL_FAST_MATH is 0 (esp-dl/dl/dl_define_private.hpp:21, dl_math.hpp:60-72) */
        const int64_t inner = d->inner > 1 ? d->inner : 1;
        for (int64_t r = 0; r < d->rows; r++) {
            const int64_t base = (r / inner) * d->len * inner + r % inner;
            float inv_norm;
            if (d->p == 1) {
                float sum_abs = 0.0f;
                for (int j = 0; j < d->len; j++) sum_abs += fabsf((float)load_int(d->input, d->dtype, base + j * inner));
                inv_norm = sum_abs > 0.0f ? 1.0f / sum_abs : 0.0f;
            } else {
                int64_t sq = 0;
                for (int j = 0; j < d->len; j++) {
                    const int64_t v = load_int(d->input, d->dtype, base + j * inner);
                    sq += v * v;
                }
                const float sum_sq = is8 ? (float)(int32_t)sq : (float)sq;
                inv_norm = sum_sq > 0.0f ? 1.0f / sqrtf(sum_sq) : 0.0f;
            }
            if (inner == 1) { /* last axis: the scale is folded into the factor first (:153-160) */
                inv_norm *= output_scale;
                for (int j = 0; j < d->len; j++) {
                    const float result = (float)load_int(d->input, d->dtype, base + j) * inv_norm;
                    store_sat(d->output, d->dtype, base + j, inv_norm > 0.0f ? fround(result, mode) : 0);
                }
            } else { /* any other axis: two multiplications (:175-181) */
                for (int j = 0; j < d->len; j++) {
                    const float result = (float)load_int(d->input, d->dtype, base + j * inner) * inv_norm;
                    store_sat(d->output, d->dtype, base + j * inner, inv_norm > 0.0f ? fround(result * output_scale, mode) : 0);
                }
            }
        }
        return ESPDL_OK;
    }
    for (int64_t i = 0; i < d->rows; i++) {
        const int64_t base = i * d->len;
        if (d->op == ESPDL_NORM_RMS) { /* esp-dl/dl/module/include/dl_module_rms_normalization.hpp:57-84, dl_base_norm.cpp:16-20 */
            const float input_scale_sq = input_scale * input_scale;
            const float scale_factor = input_scale * output_scale;
            int64_t sum_sq = 0;
            for (int j = 0; j < d->len; j++) {
                const int64_t v = load_int(d->input, d->dtype, base + j);
                sum_sq += v * v;
            }
            const float mean_sq = (is8 ? (float)(int32_t)sum_sq : (float)sum_sq) * input_scale_sq / d->len;
            float rms = 1.0f / sqrtf(mean_sq + d->epsilon); /* math::fast_inv_sqrt with DL_FAST_MATH 0, dl_math.hpp:60-72 */
            rms *= scale_factor;
            for (int j = 0; j < d->len; j++) {
                float result = (float)load_int(d->input, d->dtype, base + j) * rms;
                result *= ((const float *)d->scale)[j];
                store_sat(d->output, d->dtype, base + j, fround(result, mode));
            }
        } else { /* esp-dl/dl/module/include/dl_module_layer_normalization.hpp:141-214 */
            const float scale_scale = d->scale ? dl_scale(d->scale_exponent) : 1.0f;
            const float bias_scale = d->bias ? dl_scale(d->bias_exponent) : 0.0f;
            int sum_val = 0;
            for (int j = 0; j < d->len; j++) sum_val += (int)load_int(d->input, d->dtype, base + j);
            float mean_val = (float)(sum_val * 1.0 / d->len);
            if (d->mean)
                store_sat(d->mean, d->dtype, i, fround(mean_val * dl_rescale(d->mean_exponent) * input_scale, mode));
            float variance = 0.0f;
            for (int j = 0; j < d->len; j++) {
                const float diff = (float)load_int(d->input, d->dtype, base + j) - mean_val;
                variance += diff * diff;
            }
            mean_val *= input_scale;
            variance *= input_scale * input_scale;
            variance /= d->len;
            const float inv_std = 1.0f / oracle_sqrt_newton(variance + d->epsilon);
            if (d->inv_std_dev)
                store_sat(d->inv_std_dev, d->dtype, i, fround(inv_std * dl_rescale(d->inv_std_dev_exponent), mode));
            for (int j = 0; j < d->len; j++) {
                const float x_val = (float)load_int(d->input, d->dtype, base + j) * input_scale;
                const float normalized = (x_val - mean_val) * inv_std;
                const float scale_val = d->scale ? (float)load_int(d->scale, d->dtype, j) * scale_scale : 1.0f;
                const float bias_val = d->bias ? (float)load_int(d->bias, d->dtype, j) * bias_scale : 0.0f;
                const float result = normalized * scale_val + bias_val;
                store_sat(d->output, d->dtype, base + j, fround(result * output_scale, mode));
            }
        }
    }
    return ESPDL_OK;
}

/* ---------------------------------------------------------------- ReverseSequence, ScatterND */
/* dl::module::ReverseSequence::reverse_sequence_impl (esp-dl/dl/module/include/dl_module_reverse_sequence.hpp:14-58):
 * copy, then for every batch swap time steps t and len-1-t for t < len/2. */
int oracle_reverse_sequence(const espdl_reverse_sequence_desc *d, const int64_t *seq_lens_host)
{
    if (!d || !d->input || !d->output || !seq_lens_host)
        return ESPDL_ERR_INVALID_ARG;
    const int64_t es = d->elem_size, total = (int64_t)d->dim0 * d->dim1 * d->feature;
    memcpy(d->output, d->input, (size_t)(total * es));
    const int batch = d->batch_axis == 0 ? d->dim0 : d->dim1, time = d->batch_axis == 0 ? d->dim1 : d->dim0;
    const int64_t batch_stride = d->batch_axis == 0 ? d->dim1 * d->feature : d->feature;
    const int64_t time_stride = d->batch_axis == 0 ? d->feature : d->dim1 * d->feature;
    uint8_t *out = (uint8_t *)d->output;
    for (int b = 0; b < batch; b++) {
        const int len = (int)seq_lens_host[b];
        if (len <= 1 || len > time)
            continue;
        for (int t = 0; t < len / 2; t++) {
            uint8_t *p1 = out + (b * batch_stride + t * time_stride) * es, *p2 = out + (b * batch_stride + (len - 1 - t) * time_stride) * es;
            for (int64_t i = 0; i < d->feature * es; i++) {
                const uint8_t tmp = p1[i];
                p1[i] = p2[i];
                p2[i] = tmp;
            }
        }
    }
    return ESPDL_OK;
}

/* dl::module::ScatterND::forward_template with apply_reduction (esp-dl/dl/module/include/dl_module_scatter_nd.hpp:34-103,
 * 160-228): slices in order, add / mul saturate after every update. */
int oracle_scatter_nd(const espdl_scatter_nd_desc *d)
{
    if (!d || !d->data || !d->output)
        return ESPDL_ERR_INVALID_ARG;
    const int64_t es = d->dtype == ESPDL_DTYPE_INT8 ? 1 : (d->dtype == ESPDL_DTYPE_INT16 ? 2 : 4);
    if (d->data != d->output)
        memcpy(d->output, d->data, (size_t)(d->data_size * es));
    for (int s = 0; s < d->n_slices; s++) {
        int64_t flat = 0;
        for (int k = 0; k < d->index_depth; k++) flat += d->indices[(int64_t)s * d->index_depth + k] * d->axis_offset[k];
        if (flat < 0 || flat + d->slice_size > d->data_size)
            continue;
        for (int64_t i = 0; i < d->slice_size; i++) {
            const int64_t o = flat + i, u = (int64_t)s * d->slice_size + i;
            if (d->dtype == ESPDL_DTYPE_FLOAT) {
                float *out = (float *)d->output;
                const float cur = out[o], upd = ((const float *)d->updates)[u];
                out[o] = d->reduction == ESPDL_SCATTER_ADD ? cur + upd : d->reduction == ESPDL_SCATTER_MUL ? cur * upd
                    : d->reduction == ESPDL_SCATTER_MAX ? (cur > upd ? cur : upd) : d->reduction == ESPDL_SCATTER_MIN ? (cur < upd ? cur : upd) : upd;
            } else {
                const int64_t cur = load_int(d->output, d->dtype, o), upd = load_int(d->updates, d->dtype, u);
                const int64_t v = d->reduction == ESPDL_SCATTER_ADD ? cur + upd : d->reduction == ESPDL_SCATTER_MUL ? cur * upd
                    : d->reduction == ESPDL_SCATTER_MAX ? (cur > upd ? cur : upd) : d->reduction == ESPDL_SCATTER_MIN ? (cur < upd ? cur : upd) : upd;
                store_sat(d->output, d->dtype, o, v);
            }
        }
    }
    return ESPDL_OK;
}

/* ---------------------------------------------------------------- GRU, LSTM */
/* math::sigmoid / math::tanh (esp-dl/dl/math/include/dl_math.hpp:168-176): 1.0 / (1.0 + expf(-x)) in double, narrowed to
 * float; tanh = 2 * sigmoid(2 * x) - 1 in float. */
static float math_sigmoid(float x) { return (float)(1.0 / (1.0 + expf(-x))); }
static float math_tanh(float x) { return 2 * math_sigmoid(2 * x) - 1; }

/* Entry count - 1 of math::SigmoidLUT(e, -6.3, 6.3) (which = 0) or math::TanhLUT(e, -3.5, 3.5) (which = 1), and the table
 * itself when `table` is not NULL (esp-dl/dl/math/include/dl_math.hpp:331-352, 385-405; the bounds as the modules pass them,
 * dl_module_gru.hpp:49-50). */
int oracle_rnn_table(int gate_exponent, int which, float *table)
{
    const float bound = which == 0 ? (float)6.3 : (float)3.5; /* a double literal passed to a float parameter */
    const float input_scale = dl_scale(gate_exponent);
    int quant_min = (int)(-bound / input_scale) - 1, quant_max = (int)(bound / input_scale) + 1;
    if (-quant_min > quant_max)
        quant_max = -quant_min;
    if (table)
        for (int i = 0; i <= quant_max; i++) table[i] = which == 0 ? math_sigmoid(i * input_scale) : math_tanh(i * input_scale);
    return quant_max;
}

typedef struct {
    const float *t;
    int max;
} rnn_lut;

static float sigmoid_get(const rnn_lut *l, int index) /* SigmoidLUT::get, dl_math.hpp:360-375 */
{
    if (index >= 0)
        return index < l->max ? l->t[index] : l->t[l->max];
    return index > -l->max ? 1 - l->t[-index] : 1 - l->t[l->max];
}

static float tanh_get(const rnn_lut *l, int index) /* TanhLUT::get, dl_math.hpp:413-428 */
{
    if (index >= 0)
        return index < l->max ? l->t[index] : l->t[l->max];
    return index > -l->max ? -l->t[-index] : -l->t[l->max];
}

/* base::mat_vec_dotprod with dotprod_c (esp-dl/dl/base/dl_base_dotprod.hpp:36-43, dl_base_dotprod.cpp:8-42) */
static void rnn_mat_vec(const void *matrix, int dtype, const int32_t *vector, int16_t *result, int rows, int cols, int shift, int mode)
{
    const float scale = dl_rescale(shift);
    for (int i = 0; i < rows; i++) {
        int64_t acc = 0;
        for (int j = 0; j < cols; j++) acc += (int32_t)load_int(matrix, dtype, (int64_t)i * cols + j) * vector[j];
        const float f = dtype == ESPDL_DTYPE_INT8 ? (float)(int32_t)acc * scale : (float)acc * scale;
        result[i] = (int16_t)clamp64(fround(f, mode), -32768, 32767);
    }
}

int oracle_rnn(const espdl_rnn_desc *d)
{
    if (!d || !d->x || !d->w || !d->r || !d->y || !d->y_h || !d->sigmoid_table || !d->tanh_table)
        return ESPDL_ERR_INVALID_ARG;
    const int H = d->hidden_size, G = d->op == ESPDL_RNN_GRU ? 3 : 4, GH = G * H, mode = d->round_mode, dt = d->dtype;
    const rnn_lut sig = {d->sigmoid_table, d->sigmoid_max}, tnh = {d->tanh_table, d->tanh_max};
    int32_t *h_prev = (int32_t *)calloc((size_t)H, 4), *xv = (int32_t *)calloc((size_t)d->input_size, 4);
    int16_t *c_prev = (int16_t *)calloc((size_t)H, 2), *ic = (int16_t *)calloc((size_t)GH, 2), *hc = (int16_t *)calloc((size_t)GH, 2);
    float *gates = (float *)calloc((size_t)GH, 4);
    const float rescale_y = dl_rescale(d->y_exponent), rescale_c = dl_rescale(d->c_exponent);
    const int w_shift = d->gate_exponent - (d->x_exponent + d->w_exponent), r_shift = d->gate_exponent - (d->h_exponent + d->r_exponent);
    const int64_t lo = dt == ESPDL_DTYPE_INT8 ? -128 : -32768, hi = dt == ESPDL_DTYPE_INT8 ? 127 : 32767;
    const int es = dt == ESPDL_DTYPE_INT8 ? 1 : 2;
    for (int di = 0; di < d->directions; di++) {
        const uint8_t *w = (const uint8_t *)d->w + (int64_t)di * GH * d->input_size * es, *r = (const uint8_t *)d->r + (int64_t)di * GH * H * es;
        const int16_t *wb = d->b ? d->b + (int64_t)di * 2 * GH : NULL, *rb = wb ? wb + GH : NULL;
        for (int i = 0; i < H; i++) {
            h_prev[i] = d->initial_h ? (int32_t)load_int(d->initial_h, dt, di * H + i) : 0;
            c_prev[i] = d->initial_c ? d->initial_c[di * H + i] : 0;
        }
        for (int step = 0; step < d->seq_length; step++) {
            const int t = di == 0 ? step : d->seq_length - 1 - step; /* the reverse pass walks the pointers backwards */
            for (int i = 0; i < d->input_size; i++) xv[i] = (int32_t)load_int(d->x, dt, (int64_t)t * d->input_size + i);
            rnn_mat_vec(w, dt, xv, ic, GH, d->input_size, w_shift, mode);
            rnn_mat_vec(r, dt, h_prev, hc, GH, H, r_shift, mode);
            if (d->op == ESPDL_RNN_GRU) { /* dl_module_gru.hpp:216-242 */
                if (wb)
                    for (int i = 0; i < GH; i++) {
                        ic[i] = (int16_t)(ic[i] + wb[i]);
                        hc[i] = (int16_t)(hc[i] + rb[i]);
                    }
                for (int i = 0; i < 2 * H; i++) gates[i] = sigmoid_get(&sig, ic[i] + hc[i]);
                for (int i = 0; i < H; i++) {
                    const int index = fround(ic[i + 2 * H] + gates[H + i] * hc[i + 2 * H], mode);
                    gates[2 * H + i] = tanh_get(&tnh, index);
                }
                for (int i = 0; i < H; i++) {
                    float temp = (1 - gates[i]) * gates[2 * H + i] * rescale_y;
                    temp += gates[i] * h_prev[i];
                    h_prev[i] = (int32_t)clamp64(fround(temp, mode), lo, hi);
                }
            } else { /* dl_module_lstm.hpp:257-283 */
                for (int i = 0; i < GH; i++) ic[i] = (int16_t)(ic[i] + (wb ? wb[i] + hc[i] + rb[i] : hc[i]));
                for (int i = 0; i < H; i++) {
                    const float ig = sigmoid_get(&sig, ic[i]), og = sigmoid_get(&sig, ic[H + i]);
                    const float fg = sigmoid_get(&sig, ic[2 * H + i]), gg = tanh_get(&tnh, ic[3 * H + i]);
                    float temp = fg * c_prev[i] + ig * gg * rescale_c;
                    c_prev[i] = (int16_t)fround(temp, mode);
                    temp = og * tanh_get(&tnh, c_prev[i]) * rescale_y;
                    h_prev[i] = (int32_t)clamp64(fround(temp, mode), lo, hi);
                }
            }
            for (int i = 0; i < H; i++) store_sat(d->y, dt, ((int64_t)t * d->directions + di) * H + i, h_prev[i]);
        }
        for (int i = 0; i < H; i++) {
            store_sat(d->y_h, dt, di * H + i, h_prev[i]);
            if (d->op == ESPDL_RNN_LSTM && d->y_c)
                d->y_c[di * H + i] = c_prev[i];
        }
    }
    free(h_prev), free(xv), free(c_prev), free(ic), free(hc), free(gates);
    return ESPDL_OK;
}
