// Elementwise operators of the quantized path: Add / Sub / Mul with numpy broadcasting,
// RequantizeLinear (TensorBase::assign), 8-bit LUT activations, Clip, ReLU, PReLU.
// All are bandwidth bound.  The int8 same-shape case (what a network's residual Adds, LUT
// activations and requantize nodes are) runs a 128-bit vectorised kernel; everything else
// (broadcast operands, int16, float endpoints) runs a strided scalar kernel.
//
// Arithmetic follows the reference exactly, including its fp32 sequences:
//   Add/Sub  esp-dl/dl/base/dl_base_add.cpp:8-44      Mul   esp-dl/dl/base/dl_base_mul.cpp:9-46
//   assign   esp-dl/dl/tensor/src/dl_tensor_base.cpp:223-404
//   LUT      esp-dl/dl/base/dl_base_lut.cpp:10-15     Clip  esp-dl/dl/module/include/dl_module_clip.hpp:78-90
//   ReLU     esp-dl/dl/module/include/dl_module_relu.hpp:66-91   PReLU esp-dl/dl/base/dl_base_prelu.cpp:5-19
//   Max/Min  esp-dl/dl/base/dl_base_max.cpp, dl_base_min.cpp     Div   esp-dl/dl/base/dl_base_div.cpp:87-207
//   Mod      esp-dl/dl/base/dl_base_mod.cpp:9-62                 comparisons esp-dl/dl/base/dl_base_greater.cpp:9-44 (and siblings)
#include "common.cuh"

#include <climits>

namespace espdl {

struct EltParams {
    const void *a, *b;
    void *out;
    int op, idt, odt;
    int os[4];
    long long sa[4], sb[4]; // element strides (0 on broadcast axes)
    int e0, e1, eo, lo, hi, half_even;
    float mul_scale, clip_rescale, in_scale, in1_scale, out_rescale, inv_scale;
    int prelu_shift, lut_shift;
    const int8_t *pow_table; // Pow on int8: the host's 256 x 256 answers, or null
    int div_n1, div_table0; // Div: divisor broadcast along the innermost axis; int8 dividend of one element (table form)
    float div_scale;
    long long total;
    // rows of the innermost axis that do not follow one another in memory (channel slices of a wider tensor): element
    // strides between rows of the output / the operands; 0 = dense.  Vector kernels: the same in 16-byte units.
    long long ro, ra, rb;
    int vpr; // 16-byte units per row (vector kernels, strided rows only; 0 = flat)
    int vpr_shift; // log2(vpr) when it is a power of two, else -1
};

// Vector index -> unit offsets of the output and the two operands.
__device__ __forceinline__ void vec_offsets(const EltParams &p, long long v, long long &io, long long &ia, long long &ib)
{
    if (p.vpr) {
        // no 64-bit division on the common widths (1, 2, 4, 8 units per row)
        const long long row = p.vpr_shift >= 0 ? (v >> p.vpr_shift) : (v < 0x7fffffffll ? (long long)((unsigned)v / (unsigned)p.vpr) : v / p.vpr);
        const long long col = v - row * p.vpr;
        io = row * p.ro + col, ia = row * p.ra + col, ib = row * p.rb + col;
    } else {
        io = ia = ib = v;
    }
}

__host__ __device__ __forceinline__ bool elt_two_operands(int op)
{
    return op == ESPDL_ELT_ADD || op == ESPDL_ELT_SUB || op == ESPDL_ELT_MUL || (op >= ESPDL_ELT_MAX && op <= ESPDL_ELT_POW);
}

__device__ __forceinline__ long long ld_int(const void *p, int dt, long long i)
{
    return dt == ESPDL_DTYPE_INT8 ? (long long)((const int8_t *)p)[i] : (long long)((const int16_t *)p)[i];
}

__device__ __forceinline__ void st_sat(void *p, int dt, long long i, long long v)
{
    if (dt == ESPDL_DTYPE_INT8)
        ((int8_t *)p)[i] = (int8_t)max(-128ll, min(127ll, v));
    else if (dt == ESPDL_DTYPE_BOOL)
        ((uint8_t *)p)[i] = v != 0;
    else
        ((int16_t *)p)[i] = (int16_t)max(-32768ll, min(32767ll, v));
}

// One integer-in / integer-out element.  a, b are the widened operands.
__device__ __forceinline__ long long elt_int(const EltParams &p, long long a, long long b)
{
    switch (p.op) {
    case ESPDL_ELT_ADD: return a + b;
    case ESPDL_ELT_SUB: return a - b;
    case ESPDL_ELT_MUL: {
        const int t = (int)(a * b);
        return fround(__fmul_rn(__int2float_rn(t), p.mul_scale), p.half_even);
    }
    case ESPDL_ELT_REQUANTIZE: {
        if (p.e0 == p.eo)
            return a;
        const float tmp = __fmul_rn(__int2float_rn((int)a), p.in_scale);
        return fround(__fmul_rn(tmp, p.inv_scale), p.half_even);
    }
    case ESPDL_ELT_CLIP: {
        const long long v = max((long long)p.lo, min((long long)p.hi, a));
        return fround(__fmul_rn(__int2float_rn((int)v), p.clip_rescale), p.half_even);
    }
    case ESPDL_ELT_RELU: {
        if (p.e0 == p.eo)
            return a >= 0 ? a : 0;
        const float temp = __fmul_rn(__int2float_rn((int)a), p.in_scale);
        return temp >= 0 ? (long long)fround(__fmul_rn(temp, p.out_rescale), p.half_even) : 0ll;
    }
    case ESPDL_ELT_PRELU: {
        if (a >= 0)
            return a;
        long long prod = a * b;
        if (p.idt == ESPDL_DTYPE_INT8)
            prod = (int)prod;
        long long v = p.prelu_shift > 0 ? (prod >> p.prelu_shift) : (long long)((unsigned long long)prod << (-p.prelu_shift));
        if (p.idt == ESPDL_DTYPE_INT8)
            v = (int)v;
        return v;
    }
    case ESPDL_ELT_MAX: return max(a, b);
    case ESPDL_ELT_MIN: return min(a, b);
    case ESPDL_ELT_DIV: {
        const long long hi = p.idt == ESPDL_DTYPE_INT8 ? 127 : 32767, lo = -hi - 1;
        if (p.div_table0) // int8 dividend of one element: the reference tabulates by divisor (dl_base_div.cpp:17-31)
            return b == 0 ? (a > 0 ? hi : lo) : (long long)fround(__fdiv_rn(__fmul_rn(__int2float_rn((int)a), p.div_scale), __int2float_rn((int)b)), p.half_even);
        if (a == 0)
            return 0;
        if (b == 0)
            return a > 0 ? hi : lo;
        const float fa = __int2float_rn((int)a), fb = __int2float_rn((int)b);
        const float q = p.div_n1 ? __fmul_rn(fa, __fdiv_rn(p.div_scale, fb)) : __fdiv_rn(__fmul_rn(fa, p.div_scale), fb);
        return fround(q, p.half_even);
    }
    case ESPDL_ELT_MOD: {
        const float av = __fmul_rn(__int2float_rn((int)a), p.in_scale), bv = __fmul_rn(__int2float_rn((int)b), p.in1_scale);
        const float r = bv != 0.f ? fmodf(av, bv) : 0.f;
        return fround(__fmul_rn(r, p.out_rescale), p.half_even);
    }
    case ESPDL_ELT_POW: {
        if (p.pow_table)
            return p.pow_table[(((unsigned)a & 0xffu) ^ 0x80u) * 256u + (((unsigned)b & 0xffu) ^ 0x80u)];
        const float av = __fmul_rn(__int2float_rn((int)a), p.in_scale), bv = __fmul_rn(__int2float_rn((int)b), p.in1_scale);
        const float r = __fmul_rn(powf(av, bv), p.out_rescale);
        // a float that is no int32 (NaN, infinity, too large) converts to the minimum on x86, where the reference runs
        if (!(fabsf(r) < 2147483520.f))
            return (long long)INT_MIN;
        return fround(r, p.half_even);
    }
    case ESPDL_ELT_GREATER: return a > b;
    case ESPDL_ELT_GREATER_EQUAL: return a >= b;
    case ESPDL_ELT_EQUAL: return a == b;
    case ESPDL_ELT_LESS: return a < b;
    case ESPDL_ELT_LESS_EQUAL: return a <= b;
    default: return 0;
    }
}

__global__ void __launch_bounds__(256) elt_generic_kernel(EltParams p)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < p.total; i += (long long)gridDim.x * blockDim.x) {
        long long r = i;
        const int i0 = (int)(r % p.os[3]);
        r /= p.os[3];
        const int i1 = (int)(r % p.os[2]);
        r /= p.os[2];
        const int i2 = (int)(r % p.os[1]);
        const int i3 = (int)(r / p.os[1]);
        const long long ai = i3 * p.sa[0] + i2 * p.sa[1] + i1 * p.sa[2] + i0 * p.sa[3];
        const long long bi = i3 * p.sb[0] + i2 * p.sb[1] + i1 * p.sb[2] + i0 * p.sb[3];
        const long long oi = p.ro ? (i / p.os[3]) * p.ro + i0 : i;
        if (p.op == ESPDL_ELT_LUT && p.idt == ESPDL_DTYPE_INT16) {
            // nearest table entry: index = ((uint16)x ^ 0x8000) >> shift, rounded (dl_base_lut.cpp:50-69)
            const uint32_t value = (uint32_t)(uint16_t)((const int16_t *)p.a)[ai] ^ 0x8000u;
            uint32_t index = value;
            if (p.lut_shift > 0) {
                index = value >> p.lut_shift;
                const uint32_t rem = value & ((1u << p.lut_shift) - 1u), half = 1u << (p.lut_shift - 1);
                if (p.half_even ? (rem > half || (rem == half && (index & 1u))) : rem >= half)
                    index++;
            }
            ((int16_t *)p.out)[oi] = ((const int16_t *)p.b)[index];
        } else if (p.op == ESPDL_ELT_LUT) {
            ((int8_t *)p.out)[oi] = ((const int8_t *)p.b)[(uint8_t)((const int8_t *)p.a)[ai] ^ 0x80u];
        } else if (p.op == ESPDL_ELT_REQUANTIZE && p.idt == ESPDL_DTYPE_FLOAT) {
            st_sat(p.out, p.odt, oi, fround(__fmul_rn(((const float *)p.a)[ai], p.out_rescale), p.half_even));
        } else if (p.op == ESPDL_ELT_REQUANTIZE && p.odt == ESPDL_DTYPE_FLOAT) {
            ((float *)p.out)[oi] = __fmul_rn(__int2float_rn((int)ld_int(p.a, p.idt, ai)), p.in_scale);
        } else {
            const long long a = ld_int(p.a, p.idt, ai);
            long long b = 0;
            if (elt_two_operands(p.op))
                b = ld_int(p.b, p.idt, bi);
            else if (p.op == ESPDL_ELT_PRELU)
                b = ld_int(p.b, p.idt, i0);
            st_sat(p.out, p.odt, oi, elt_int(p, a, b));
        }
    }
}

// int8 -> int8, operands of identical shape, 16 elements per thread.
template <int OP>
__global__ void __launch_bounds__(256) elt_s8_vec16_kernel(EltParams p, long long nvec)
{
    __shared__ int8_t table[256];
    // One-operand int8 -> int8 operators are functions of the input byte: every block tabulates the operator once with
    // the scalar code (so the rounding is the reference's) and then runs as a table lookup like LUT itself.
    constexpr bool TABULATED = OP == ESPDL_ELT_REQUANTIZE || OP == ESPDL_ELT_CLIP || OP == ESPDL_ELT_RELU;
    if (OP == ESPDL_ELT_LUT) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) table[i] = ((const int8_t *)p.b)[i];
        __syncthreads();
    } else if (TABULATED) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) {
            EltParams q2 = p;
            q2.op = OP;
            const int a = (int)(int8_t)(uint8_t)(i ^ 0x80);
            table[i] = (int8_t)sat8((int)max(-1000000ll, min(1000000ll, elt_int(q2, a, 0))));
        }
        __syncthreads();
    }
    for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
        long long io, ia, ib;
        vec_offsets(p, v, io, ia, ib);
        const uint4 a4 = ((const uint4 *)p.a)[ia];
        uint4 b4 = make_uint4(0, 0, 0, 0);
        if (elt_two_operands(OP))
            b4 = ((const uint4 *)p.b)[ib];
        const uint32_t aw[4] = {a4.x, a4.y, a4.z, a4.w};
        const uint32_t bw[4] = {b4.x, b4.y, b4.z, b4.w};
        uint32_t ow[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            uint32_t wd = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int a = (int)(int8_t)(aw[q] >> (8 * j));
                const int b = (int)(int8_t)(bw[q] >> (8 * j));
                int r;
                if (OP == ESPDL_ELT_LUT || TABULATED) {
                    r = table[(uint8_t)a ^ 0x80u];
                } else if (OP == ESPDL_ELT_ADD) {
                    r = sat8(a + b);
                } else if (OP == ESPDL_ELT_SUB) {
                    r = sat8(a - b);
                } else {
                    EltParams q2 = p;
                    q2.op = OP;
                    r = sat8((int)max(-1000000ll, min(1000000ll, elt_int(q2, a, b))));
                }
                wd |= ((uint32_t)r & 0xffu) << (8 * j);
            }
            ow[q] = wd;
        }
        ((uint4 *)p.out)[io] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

// int8 (op) one-element int8 -> int8 (Mul by a scalar factor, Add of a constant, ...): with the second operand fixed the
// operator is a function of the input byte, so every block tabulates it once with the scalar code (the reference's
// rounding, whatever the operator) and then runs as a table lookup at the speed of LUT.
__global__ void __launch_bounds__(256) elt_s8_scalar_b_kernel(EltParams p, long long nvec)
{
    __shared__ int8_t table[256];
    const int b = (int)((const int8_t *)p.b)[0];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
        const int a = (int)(int8_t)(uint8_t)(i ^ 0x80);
        table[i] = (int8_t)sat8((int)max(-1000000ll, min(1000000ll, elt_int(p, a, b))));
    }
    __syncthreads();
    for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
        long long io, ia, ib;
        vec_offsets(p, v, io, ia, ib);
        const uint4 a4 = ((const uint4 *)p.a)[ia];
        const uint32_t aw[4] = {a4.x, a4.y, a4.z, a4.w};
        uint32_t ow[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            uint32_t wd = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) wd |= ((uint32_t)(uint8_t)table[(uint8_t)(aw[q] >> (8 * j)) ^ 0x80u]) << (8 * j);
            ow[q] = wd;
        }
        ((uint4 *)p.out)[io] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

template <int OP>
static void launch_vec(const EltParams &p, long long nvec, cudaStream_t s)
{
    const int threads = 256;
    long long blocks = min((nvec + threads - 1) / threads, (long long)num_sms() * 16);
    elt_s8_vec16_kernel<OP><<<(unsigned)max(blocks, 1ll), threads, 0, s>>>(p, nvec);
}

} // namespace espdl

using namespace espdl;

extern "C" int espdl_b200_eltwise(const espdl_eltwise_desc *d, void *stream)
{
    if (!d || !d->input0 || !d->output || d->ndim < 1 || d->ndim > 4)
        return ESPDL_ERR_INVALID_ARG;
    const bool binary = elt_two_operands(d->op);
    const bool compare = d->op >= ESPDL_ELT_GREATER && d->op <= ESPDL_ELT_LESS_EQUAL;
    if ((binary || d->op == ESPDL_ELT_LUT || d->op == ESPDL_ELT_PRELU) && !d->input1)
        return ESPDL_ERR_INVALID_ARG;
    if (d->op < ESPDL_ELT_ADD || d->op > ESPDL_ELT_POW)
        return ESPDL_ERR_INVALID_ARG;
    auto is_int = [](int t) { return t == ESPDL_DTYPE_INT8 || t == ESPDL_DTYPE_INT16; };
    if (d->op == ESPDL_ELT_REQUANTIZE) {
        const bool ok = (is_int(d->in_dtype) || d->in_dtype == ESPDL_DTYPE_FLOAT) && (is_int(d->out_dtype) || d->out_dtype == ESPDL_DTYPE_FLOAT) &&
            !(d->in_dtype == ESPDL_DTYPE_FLOAT && d->out_dtype == ESPDL_DTYPE_FLOAT);
        if (!ok)
            return ESPDL_ERR_UNSUPPORTED;
    } else if (d->op == ESPDL_ELT_LUT) {
        if (d->in_dtype != d->out_dtype || !is_int(d->in_dtype) || d->lut_shift < 0 || d->lut_shift > 15)
            return ESPDL_ERR_UNSUPPORTED;
    } else if (compare) {
        if (!is_int(d->in_dtype) || d->out_dtype != ESPDL_DTYPE_BOOL)
            return ESPDL_ERR_UNSUPPORTED;
    } else if (!is_int(d->in_dtype) || d->in_dtype != d->out_dtype) {
        return ESPDL_ERR_UNSUPPORTED;
    }
    EltParams p;
    memset(&p, 0, sizeof(p));
    int os[4] = {1, 1, 1, 1}, s0[4] = {1, 1, 1, 1}, s1[4] = {1, 1, 1, 1};
    for (int i = 0; i < d->ndim; i++) {
        os[4 - d->ndim + i] = d->out_shape[i];
        s0[4 - d->ndim + i] = d->in0_shape[i];
        s1[4 - d->ndim + i] = binary ? d->in1_shape[i] : 1;
    }
    long long a = 1, b = 1, total = 1;
    bool same = true;
    // strided rows: a stride is given for a tensor whose innermost extent is the output's (no broadcast along it)
    const long long rs0 = d->in0_row_stride, rs1 = binary ? d->in1_row_stride : 0, rso = d->out_row_stride;
    if (rs0 < 0 || rs1 < 0 || rso < 0 || (rs0 && (rs0 < s0[3] || s0[3] != os[3])) || (rs1 && (rs1 < s1[3] || s1[3] != os[3])) || (rso && rso < os[3]))
        return ESPDL_ERR_INVALID_ARG;
    for (int i = 3; i >= 0; i--) {
        if (os[i] < 0 || (s0[i] != os[i] && s0[i] != 1) || (s1[i] != os[i] && s1[i] != 1))
            return ESPDL_ERR_INVALID_ARG;
        p.os[i] = os[i];
        p.sa[i] = s0[i] == 1 ? 0 : a;
        p.sb[i] = s1[i] == 1 ? 0 : b;
        a *= i == 3 && rs0 ? rs0 : s0[i], b *= i == 3 && rs1 ? rs1 : s1[i], total *= os[i];
        if (s0[i] != os[i] || (binary && s1[i] != os[i]))
            same = false;
    }
    if (total == 0)
        return ESPDL_OK;
    const bool strided = rs0 || rs1 || rso;
    if (strided && d->op == ESPDL_ELT_DIV)
        return ESPDL_ERR_UNSUPPORTED; // Div reads the operands' element counts
    p.ro = rso;
    const bool rows16 = !strided || (os[3] % 16 == 0 && rs0 % 16 == 0 && rs1 % 16 == 0 && rso % 16 == 0);
    if (strided && rows16) {
        p.vpr = os[3] / 16;
        p.vpr_shift = -1;
        for (int sft = 0; sft < 16; sft++)
            if ((1 << sft) == p.vpr)
                p.vpr_shift = sft;
        p.ra = (rs0 ? rs0 : os[3]) / 16, p.rb = (rs1 ? rs1 : os[3]) / 16;
    }
    p.a = d->input0, p.b = d->input1, p.out = d->output;
    p.op = d->op, p.idt = d->in_dtype, p.odt = d->out_dtype;
    p.e0 = d->in0_exponent, p.e1 = d->in1_exponent, p.eo = d->out_exponent;
    p.lo = d->clip_lo, p.hi = d->clip_hi, p.half_even = d->round_mode == ESPDL_ROUND_HALF_EVEN;
    p.lut_shift = d->lut_shift;
    p.pow_table = d->op == ESPDL_ELT_POW && d->in_dtype == ESPDL_DTYPE_INT8 ? (const int8_t *)d->table : nullptr;
    for (int e : {p.e0, p.e1, p.eo})
        if (e > 30 || e < -30)
            return ESPDL_ERR_INVALID_ARG;
    p.mul_scale = dl_scale(p.e0) * dl_scale(p.e1) * dl_rescale(p.eo);
    p.clip_rescale = dl_scale(p.e0) * dl_rescale(p.eo);
    p.in_scale = dl_scale(p.e0);
    p.in1_scale = dl_scale(p.e1);
    if (d->op == ESPDL_ELT_DIV) {
        // which operand the reference sees as a scalar along the innermost merged axis (dl_base_elemwise.cpp:38-100,
        // dl_base_div.cpp:208-250): that is the innermost axis on which the output is longer than 1
        int ax = 3;
        while (ax > 0 && os[ax] == 1) ax--;
        const bool in0_1 = s0[ax] == 1, in1_1 = s1[ax] == 1;
        p.div_table0 = d->in_dtype == ESPDL_DTYPE_INT8 && a == 1; // a = element count of input0 here
        p.div_n1 = d->in_dtype == ESPDL_DTYPE_INT8 ? (in1_1 && !in0_1) : in1_1;
        p.div_scale = dl_rescale(p.eo) * dl_scale(p.e0) / dl_scale(p.e1); // dl_base_div.cpp:66
    }
    p.out_rescale = dl_rescale(p.eo);
    p.inv_scale = (float)(1.0 / (double)dl_scale(p.eo));
    p.prelu_shift = p.eo - p.e0 - p.e1;
    p.total = total;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = same && rows16 && d->in_dtype == ESPDL_DTYPE_INT8 && (d->out_dtype == ESPDL_DTYPE_INT8 || compare) && total % 16 == 0 &&
        ((uintptr_t)d->input0 % 16) == 0 && ((uintptr_t)d->output % 16) == 0 && (!binary || ((uintptr_t)d->input1 % 16) == 0) &&
        d->op != ESPDL_ELT_PRELU && d->op != ESPDL_ELT_POW;
    // second operand of one element, first operand of the output's shape
    bool a_full = true;
    for (int i = 0; i < 4; i++) a_full = a_full && s0[i] == os[i];
    const bool scalar_b = binary && !compare && !same && a_full && b == 1 && rows16 && d->in_dtype == ESPDL_DTYPE_INT8 && d->out_dtype == ESPDL_DTYPE_INT8 &&
        total % 16 == 0 && ((uintptr_t)d->input0 % 16) == 0 && ((uintptr_t)d->output % 16) == 0 && d->op != ESPDL_ELT_POW;
    if ((scalar_b || vec) && p.vpr)
        p.ro = (rso ? rso : os[3]) / 16;
    if (scalar_b) {
        const long long nvec = total / 16;
        const long long blocks = min((nvec + 255) / 256, (long long)num_sms() * 16);
        elt_s8_scalar_b_kernel<<<(unsigned)max(blocks, 1ll), 256, 0, s>>>(p, nvec);
    } else if (vec) {
        const long long nvec = total / 16;
        switch (d->op) {
        case ESPDL_ELT_ADD: launch_vec<ESPDL_ELT_ADD>(p, nvec, s); break;
        case ESPDL_ELT_SUB: launch_vec<ESPDL_ELT_SUB>(p, nvec, s); break;
        case ESPDL_ELT_MUL: launch_vec<ESPDL_ELT_MUL>(p, nvec, s); break;
        case ESPDL_ELT_REQUANTIZE: launch_vec<ESPDL_ELT_REQUANTIZE>(p, nvec, s); break;
        case ESPDL_ELT_LUT: launch_vec<ESPDL_ELT_LUT>(p, nvec, s); break;
        case ESPDL_ELT_CLIP: launch_vec<ESPDL_ELT_CLIP>(p, nvec, s); break;
        case ESPDL_ELT_RELU: launch_vec<ESPDL_ELT_RELU>(p, nvec, s); break;
        case ESPDL_ELT_MAX: launch_vec<ESPDL_ELT_MAX>(p, nvec, s); break;
        case ESPDL_ELT_MIN: launch_vec<ESPDL_ELT_MIN>(p, nvec, s); break;
        case ESPDL_ELT_DIV: launch_vec<ESPDL_ELT_DIV>(p, nvec, s); break;
        case ESPDL_ELT_MOD: launch_vec<ESPDL_ELT_MOD>(p, nvec, s); break;
        case ESPDL_ELT_GREATER: launch_vec<ESPDL_ELT_GREATER>(p, nvec, s); break;
        case ESPDL_ELT_GREATER_EQUAL: launch_vec<ESPDL_ELT_GREATER_EQUAL>(p, nvec, s); break;
        case ESPDL_ELT_EQUAL: launch_vec<ESPDL_ELT_EQUAL>(p, nvec, s); break;
        case ESPDL_ELT_LESS: launch_vec<ESPDL_ELT_LESS>(p, nvec, s); break;
        case ESPDL_ELT_LESS_EQUAL: launch_vec<ESPDL_ELT_LESS_EQUAL>(p, nvec, s); break;
        default: return ESPDL_ERR_UNSUPPORTED;
        }
    } else {
        const int threads = 256;
        long long blocks = min((total + threads - 1) / threads, (long long)num_sms() * 32);
        elt_generic_kernel<<<(unsigned)blocks, threads, 0, s>>>(p);
    }
    count_launch();
    return check_launch("eltwise");
}
