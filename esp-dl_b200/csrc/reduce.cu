// Reductions over any set of axes of an int8 / int16 tensor: ReduceMean, ReduceSum, ReduceMax, ReduceMin, ReduceL1,
// ReduceSumSquare, ReduceL2 (dl_module_reduce_l1.hpp, dl_module_reduce_sum_square.hpp, dl_module_reduce_l2.hpp), ReduceProd,
// ReduceLogSum, ReduceLogSumExp (dl_module_reduce_prod.hpp, dl_module_reduce_log_sum.hpp, dl_module_reduce_log_sum_exp.hpp).
// Replaces dl::module::ReduceBase::forward_template and the reduce functions of the modules built on it
// (esp-dl/dl/module/include/dl_module_reduce_base.hpp:121-262, dl_module_reduce_mean.hpp:17-45, dl_module_reduce_sum.hpp:
// 17-42).  A thread owns one output element and walks the reduced axes; with channels innermost and kept (the usual
// spatial mean of an NHWC map) neighbouring threads read neighbouring bytes.  Integer sums are exact, so the order
// of the walk does not matter; the mean's fp32 expression is evaluated in the reference's order.  The floating-point
// accumulations (the product, the sum of exponentials) are not associative: the walk visits the reduced elements in
// the reference's order (row-major over the reduced axes), one thread per output.
#include "common.cuh"

#include <climits>

namespace espdl {

namespace {

struct ReduceParams {
    const void *in;
    void *out;
    int op, half_even, e_in, e_out;
    int nk, nr;            // kept / reduced axes
    int ksize[6], rsize[6];
    long long kstride[6], rstride[6];
    long long outputs, count;
    const float *exp_table;
};

// tool::round of a float that may be no int32 (NaN, infinity): such a value converts to the minimum on x86
__device__ __forceinline__ long long fround_x86(float v, int half_even)
{
    if (!(fabsf(v) < 2147483520.f))
        return (long long)INT_MIN;
    return fround(v, half_even);
}

template <typename T, typename ACC>
__global__ void __launch_bounds__(256) reduce_kernel(ReduceParams p)
{
    const T *in = (const T *)p.in;
    T *out = (T *)p.out;
    const int lo = sizeof(T) == 1 ? -128 : -32768, hi = sizeof(T) == 1 ? 127 : 32767;
    for (long long o = blockIdx.x * (long long)blockDim.x + threadIdx.x; o < p.outputs; o += (long long)gridDim.x * blockDim.x) {
        long long base = 0, rem = o;
        for (int k = p.nk - 1; k >= 0; k--) {
            base += (rem % p.ksize[k]) * p.kstride[k];
            rem /= p.ksize[k];
        }
        int idx[6] = {0, 0, 0, 0, 0, 0};
        long long off = base;
        ACC acc = p.op == ESPDL_REDUCE_MAX ? (ACC)lo : (p.op == ESPDL_REDUCE_MIN ? (ACC)hi : (ACC)0);
        float facc = p.op == ESPDL_REDUCE_PROD ? 1.f : 0.f; // int8 product, both sums of exponentials
        double dacc = 1.0;                                   // int16 product
        const float in_scale = dl_scale(p.e_in);
        for (long long i = 0; i < p.count; i++) {
            const ACC v = (ACC)in[off];
            if (p.op == ESPDL_REDUCE_PROD) {
                const float t = __fmul_rn((float)(int)v, in_scale);
                if (sizeof(T) == 1)
                    facc = __fmul_rn(facc, t);
                else
                    dacc = __dmul_rn(dacc, (double)t);
            } else if (p.op == ESPDL_REDUCE_LOG_SUM_EXP) {
                facc = __fadd_rn(facc, sizeof(T) == 1 ? p.exp_table[(int)v + 128] : expf(__fmul_rn((float)(int)v, in_scale)));
            } else if (p.op == ESPDL_REDUCE_MAX)
                acc = acc > v ? acc : v;
            else if (p.op == ESPDL_REDUCE_MIN)
                acc = acc < v ? acc : v;
            else if (p.op == ESPDL_REDUCE_L1)
                acc += v < 0 ? -v : v;
            else if (p.op == ESPDL_REDUCE_SUM_SQUARE || p.op == ESPDL_REDUCE_L2)
                acc += (ACC)((int)v * (int)v);
            else
                acc += v;
            for (int r = p.nr - 1; r >= 0; r--) { // odometer over the reduced axes
                off += p.rstride[r];
                if (++idx[r] < p.rsize[r])
                    break;
                off -= (long long)p.rsize[r] * p.rstride[r];
                idx[r] = 0;
            }
        }
        long long q;
        if (p.op == ESPDL_REDUCE_MEAN) {
            // tool::round(tmp * input_scale / count * output_scale), all in fp32
            float f = __fmul_rn((float)acc, dl_scale(p.e_in));
            f = __fdiv_rn(f, (float)(unsigned long long)p.count);
            f = __fmul_rn(f, dl_rescale(p.e_out));
            q = fround(f, p.half_even);
        } else if (p.op == ESPDL_REDUCE_L2) {
            // math::sqrt_newton (dl_math.hpp:83-97): r = (r + x / r) * 0.5 until |r - last| <= 1e-5, every step rounded to fp32
            const float x = __fmul_rn(sizeof(ACC) == 4 ? __int2float_rn((int)acc) : __ll2float_rn((long long)acc), dl_scale(2 * p.e_in));
            float r = x;
            if (x != 0.f) {
                for (int it = 0; it < 100; it++) {
                    const float last = r;
                    r = __fmul_rn(__fadd_rn(last, __fdiv_rn(x, last)), 0.5f);
                    if (!(fabsf(__fsub_rn(r, last)) > 0.00001f))
                        break;
                }
            }
            q = fround(__fmul_rn(r, dl_rescale(p.e_out)), p.half_even);
        } else if (p.op == ESPDL_REDUCE_PROD) {
            if (sizeof(T) == 1) {
                q = fround_x86(__fmul_rn(facc, dl_rescale(p.e_out)), p.half_even);
            } else {
                // the fp64 product times the fp32 scale, rounded as a double (floor(v + 0.5), or to nearest even)
                const double v = __dmul_rn(dacc, (double)dl_rescale(p.e_out));
                q = !(fabs(v) < 2147483647.0) ? (long long)INT_MIN : (p.half_even ? (long long)__double2ll_rn(v) : (long long)floor(__dadd_rn(v, 0.5)));
            }
        } else if (p.op == ESPDL_REDUCE_LOG_SUM) {
            // static_cast<float>(sum * input_scale): the integer sum becomes a float before the multiplication
            const float sumf = sizeof(ACC) == 4 ? __int2float_rn((int)acc) : __ll2float_rn((long long)acc);
            q = fround_x86(__fmul_rn(logf(__fmul_rn(sumf, in_scale)), dl_rescale(p.e_out)), p.half_even);
        } else if (p.op == ESPDL_REDUCE_LOG_SUM_EXP) {
            q = fround_x86(__fmul_rn(logf(facc), dl_rescale(p.e_out)), p.half_even);
        } else if (p.op == ESPDL_REDUCE_SUM || p.op == ESPDL_REDUCE_L1 || p.op == ESPDL_REDUCE_SUM_SQUARE) {
            const int shift = max(-62, min(62, p.e_out - (p.op == ESPDL_REDUCE_SUM_SQUARE ? 2 * p.e_in : p.e_in)));
            q = sizeof(ACC) == 4 ? (long long)shift_round32((int32_t)acc, max(-31, min(31, shift)), p.half_even)
                                 : shift_round64((long long)acc, shift, p.half_even);
        } else {
            q = (long long)acc;
        }
        out[o] = (T)max((long long)lo, min((long long)hi, q));
    }
}

} // namespace

int reduce_op(const espdl_reduce_desc &d, cudaStream_t s)
{
    if (!d.input || !d.output || d.ndim < 1 || d.ndim > 6 || d.op < 0 || d.op > ESPDL_REDUCE_LOG_SUM_EXP)
        return ESPDL_ERR_INVALID_ARG;
    if (d.op == ESPDL_REDUCE_LOG_SUM_EXP && d.dtype == ESPDL_DTYPE_INT8 && !d.exp_table)
        return ESPDL_ERR_INVALID_ARG;
    if (d.dtype != ESPDL_DTYPE_INT8 && d.dtype != ESPDL_DTYPE_INT16)
        return ESPDL_ERR_UNSUPPORTED;
    ReduceParams p;
    p.in = d.input, p.out = d.output, p.op = d.op, p.half_even = d.round_mode == ESPDL_ROUND_HALF_EVEN;
    p.e_in = d.in_exponent, p.e_out = d.out_exponent;
    p.exp_table = d.exp_table;
    p.nk = p.nr = 0, p.outputs = 1, p.count = 1;
    long long stride = 1;
    long long strides[6];
    for (int i = d.ndim - 1; i >= 0; i--) {
        if (d.shape[i] <= 0)
            return ESPDL_ERR_INVALID_ARG;
        strides[i] = stride;
        stride *= d.shape[i];
    }
    for (int i = 0; i < d.ndim; i++) {
        if (d.reduce[i]) {
            p.rsize[p.nr] = d.shape[i], p.rstride[p.nr] = strides[i], p.nr++;
            p.count *= d.shape[i];
        } else {
            p.ksize[p.nk] = d.shape[i], p.kstride[p.nk] = strides[i], p.nk++;
            p.outputs *= d.shape[i];
        }
    }
    if (abs(p.e_in) > 30 || abs(p.e_out) > 30)
        return ESPDL_ERR_UNSUPPORTED;
    const long long blocks = (p.outputs + 255) / 256;
    const int grid = (int)(blocks < (long long)num_sms() * 8 ? blocks : (long long)num_sms() * 8);
    if (d.dtype == ESPDL_DTYPE_INT8)
        reduce_kernel<int8_t, int32_t><<<grid, 256, 0, s>>>(p);
    else
        reduce_kernel<int16_t, long long><<<grid, 256, 0, s>>>(p);
    count_launch();
    return check_launch("reduce");
}


// ------------------------------------------------------------------------------------------ Pad
// dl::module::Pad (esp-dl/dl/module/include/dl_module_pad.hpp:10-100; per-axis rules of esp-dl/dl/base/dl_base_pad.cpp:18-66).
namespace {

struct PadParams {
    const void *in;
    void *out;
    int ndim, mode;
    int ishape[6], oshape[6], begin[6];
    long long istride[6];
    long long total;
    long long constant;
};

template <typename T>
__global__ void __launch_bounds__(256) pad_kernel(PadParams p)
{
    const T *in = (const T *)p.in;
    T *out = (T *)p.out;
    for (long long o = blockIdx.x * (long long)blockDim.x + threadIdx.x; o < p.total; o += (long long)gridDim.x * blockDim.x) {
        long long rem = o, off = 0;
        bool inside = true;
        for (int k = p.ndim - 1; k >= 0; k--) {
            int i = (int)(rem % p.oshape[k]) - p.begin[k];
            rem /= p.oshape[k];
            const int n = p.ishape[k];
            if (i < 0 || i >= n) {
                if (p.mode == ESPDL_PAD_CONSTANT)
                    inside = false;
                else if (p.mode == ESPDL_PAD_EDGE)
                    i = i < 0 ? 0 : n - 1;
                else
                    i = i < 0 ? -i : 2 * (n - 1) - i; // mirror, the edge element is not repeated
                i = max(0, min(n - 1, i));
            }
            off += (long long)i * p.istride[k];
        }
        out[o] = inside ? in[off] : (T)p.constant;
    }
}

} // namespace

int pad_op(const espdl_pad_desc &d, cudaStream_t s)
{
    if (!d.input || !d.output || d.ndim < 1 || d.ndim > 6 || d.mode < 0 || d.mode > 2)
        return ESPDL_ERR_INVALID_ARG;
    if (d.elem_size != 1 && d.elem_size != 2 && d.elem_size != 4)
        return ESPDL_ERR_UNSUPPORTED;
    PadParams p;
    p.in = d.input, p.out = d.output, p.ndim = d.ndim, p.mode = d.mode, p.constant = d.constant, p.total = 1;
    long long stride = 1;
    for (int i = d.ndim - 1; i >= 0; i--) {
        if (d.shape[i] <= 0 || d.pad_begin[i] < 0 || d.pad_end[i] < 0)
            return ESPDL_ERR_INVALID_ARG;
        if (d.mode == ESPDL_PAD_REFLECT && (d.pad_begin[i] >= d.shape[i] || d.pad_end[i] >= d.shape[i]))
            return ESPDL_ERR_INVALID_ARG;
        p.ishape[i] = d.shape[i], p.begin[i] = d.pad_begin[i], p.oshape[i] = d.shape[i] + d.pad_begin[i] + d.pad_end[i];
        p.istride[i] = stride;
        stride *= d.shape[i];
        p.total *= p.oshape[i];
    }
    const long long blocks = (p.total + 255) / 256;
    const int grid = (int)(blocks < (long long)num_sms() * 16 ? blocks : (long long)num_sms() * 16);
    if (d.elem_size == 1)
        pad_kernel<int8_t><<<grid, 256, 0, s>>>(p);
    else if (d.elem_size == 2)
        pad_kernel<int16_t><<<grid, 256, 0, s>>>(p);
    else
        pad_kernel<int32_t><<<grid, 256, 0, s>>>(p);
    count_launch();
    return check_launch("pad");
}

} // namespace espdl
