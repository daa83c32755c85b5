/*
 * ref_harness.cpp - TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * C entry points around the UNMODIFIED reference operators.  The reference's own
 * sources are compiled where they lie in the reference checkout (see the
 * Makefile beside this file) for the host CPU with no CONFIG_IDF_TARGET_*
 * defined, i.e. its generic C kernels with round-half-up; this file only builds
 * dl::TensorBase views over the caller's host buffers, instantiates the
 * reference's dl::module::* classes through their public constructors and calls
 * Module::run().  Descriptors are the same structs the CUDA backend's C ABI
 * takes, with HOST pointers.
 *
 * What the reference cannot do and this harness therefore rejects:
 *  - per-channel filter exponents (no working branch in the generic C epilogue);
 *  - HALF_EVEN rounding (a compile-time switch tied to the ESP32-P4 target);
 *  - a fused LUT in the conv epilogue, pixel strides other than dense.
 * A batch extent n > 1 is executed as n independent single-image calls, which
 * is how a caller of the reference has to run a batch (its conv / pool / resize
 * kernels read one image).
 */
#include "../include/espdl_b200.h"

#include "dl_detect_yolo11_postprocessor.hpp"
#include "dl_image_norm_quant.hpp"
#include "dl_module_add.hpp"
#include "dl_module_average_pool.hpp"
#include "dl_module_clip.hpp"
#include "dl_module_concat.hpp"
#include "dl_module_conv.hpp"
#include "dl_module_depth_to_space.hpp"
#include "dl_module_div.hpp"
#include "dl_module_equal.hpp"
#include "dl_module_greater.hpp"
#include "dl_module_greater_or_equal.hpp"
#include "dl_module_gru.hpp"
#include "dl_module_less.hpp"
#include "dl_module_less_or_equal.hpp"
#include "dl_module_gather.hpp"
#include "dl_module_gemm.hpp"
#include "dl_module_insert_zeros.hpp"
#include "dl_module_layer_normalization.hpp"
#include "dl_module_log_softmax.hpp"
#include "dl_module_lp_normalization.hpp"
#include "dl_module_lstm.hpp"
#include "dl_module_global_average_pool.hpp"
#include "dl_module_lut.hpp"
#include "dl_module_matmul.hpp"
#include "dl_module_max.hpp"
#include "dl_module_max_pool.hpp"
#include "dl_module_min.hpp"
#include "dl_module_mod.hpp"
#include "dl_module_mul.hpp"
#include "dl_module_pad.hpp"
#include "dl_module_pow.hpp"
#include "dl_module_prelu.hpp"
#include "dl_module_reduce_l1.hpp"
#include "dl_module_reduce_l2.hpp"
#include "dl_module_reduce_log_sum.hpp"
#include "dl_module_reduce_log_sum_exp.hpp"
#include "dl_module_reduce_max.hpp"
#include "dl_module_reduce_mean.hpp"
#include "dl_module_reduce_min.hpp"
#include "dl_module_reduce_prod.hpp"
#include "dl_module_reduce_sum.hpp"
#include "dl_module_reduce_sum_square.hpp"
#include "dl_module_relu.hpp"
#include "dl_module_requantize_linear.hpp"
#include "dl_module_resize.hpp"
#include "dl_module_reverse_sequence.hpp"
#include "dl_module_rms_normalization.hpp"
#include "dl_module_scatter_nd.hpp"
#include "dl_module_softmax.hpp"
#include "dl_module_space_to_depth.hpp"
#include "dl_module_sub.hpp"

#include <memory>
#include <vector>

#if defined(_OPENMP)
#include <omp.h>
#endif

using namespace dl;

static dtype_t to_dtype(int d) { return (dtype_t)d; }
static quant_type_t to_quant(int d)
{
    return d == ESPDL_DTYPE_INT8 ? QUANT_TYPE_SYMM_8BIT : d == ESPDL_DTYPE_INT16 ? QUANT_TYPE_SYMM_16BIT : QUANT_TYPE_FLOAT32;
}
static size_t esize(int d) { return d == ESPDL_DTYPE_INT8 || d == ESPDL_DTYPE_BOOL ? 1 : d == ESPDL_DTYPE_INT16 ? 2 : d == ESPDL_DTYPE_INT64 ? 8 : 4; }

static TensorBase *view(std::vector<int> shape, const void *p, int exponent, int dtype)
{
    return new TensorBase(shape, p, exponent, to_dtype(dtype), false);
}

extern "C" {

int ref_num_threads(void)
{
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* dl::module::Conv (group 1 or depthwise).  gemm != 0 routes through dl::module::Gemm with
 * input [in_w, in_c] instead (requires n = in_h = kh = kw = 1). */
int ref_conv2d(const espdl_conv_desc *d, int gemm)
{
    if (!d || d->per_channel || d->lut || d->round_mode != ESPDL_ROUND_HALF_UP)
        return ESPDL_ERR_UNSUPPORTED;
    if ((d->in_pixel_stride && d->in_pixel_stride != d->in_c) || (d->out_pixel_stride && d->out_pixel_stride != d->out_c))
        return ESPDL_ERR_UNSUPPORTED;
    const size_t es = esize(d->dtype);
    const quant_type_t qt = to_quant(d->dtype);
    const int bias_dtype = d->dtype == ESPDL_DTYPE_INT8 ? ESPDL_DTYPE_INT32 : ESPDL_DTYPE_INT64;
    const int dw = d->group != 1;
    std::vector<int> fshape = dw ? std::vector<int>{d->kh, d->kw, d->in_c, 1} : std::vector<int>{d->kh, d->kw, d->in_c, d->out_c};
    const size_t in_img = (size_t)d->in_h * d->in_w * d->in_c * es, out_img = (size_t)d->out_h * d->out_w * d->out_c * es;
    int status = ESPDL_OK;
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
    for (int n = 0; n < d->n; n++) {
        std::unique_ptr<TensorBase> filter(view(fshape, d->filter, d->filter_exponent, d->dtype));
        std::unique_ptr<TensorBase> bias(d->bias ? view({d->out_c}, d->bias, d->in_exponent + d->filter_exponent, bias_dtype) : nullptr);
        const char *ip = (const char *)d->input + (size_t)n * in_img;
        char *op = (char *)d->output + (size_t)n * out_img;
        if (gemm) {
            std::unique_ptr<TensorBase> in(view({d->in_w, d->in_c}, ip, d->in_exponent, d->dtype));
            std::unique_ptr<TensorBase> out(view({d->out_w, d->out_c}, op, d->out_exponent, d->dtype));
            module::Gemm m((activation_type_t)d->activation, nullptr, qt);
            std::vector<TensorBase *> ins = {in.get(), filter.get()};
            if (bias)
                ins.push_back(bias.get());
            m.run(ins, {out.get()}, RUNTIME_MODE_SINGLE_CORE);
        } else {
            std::unique_ptr<TensorBase> in(view({1, d->in_h, d->in_w, d->in_c}, ip, d->in_exponent, d->dtype));
            std::unique_ptr<TensorBase> out(view({1, d->out_h, d->out_w, d->out_c}, op, d->out_exponent, d->dtype));
            module::Conv m((activation_type_t)d->activation,
                           {d->pad_top, d->pad_bottom, d->pad_left, d->pad_right},
                           {d->dilation_h, d->dilation_w},
                           {d->stride_h, d->stride_w},
                           nullptr,
                           d->group,
                           qt);
            std::vector<TensorBase *> ins = {in.get(), filter.get()};
            if (bias)
                ins.push_back(bias.get());
            m.run(ins, {out.get()}, RUNTIME_MODE_SINGLE_CORE);
        }
    }
    return status;
}

int ref_eltwise(const espdl_eltwise_desc *d)
{
    if (!d || d->round_mode != ESPDL_ROUND_HALF_UP)
        return ESPDL_ERR_UNSUPPORTED;
    std::vector<int> os(d->out_shape, d->out_shape + d->ndim), s0(d->in0_shape, d->in0_shape + d->ndim),
        s1(d->in1_shape, d->in1_shape + d->ndim);
    const quant_type_t qt = to_quant(d->in_dtype == ESPDL_DTYPE_FLOAT ? d->out_dtype : d->in_dtype);
    std::unique_ptr<TensorBase> in0(view(s0, d->input0, d->in0_exponent, d->in_dtype));
    std::unique_ptr<TensorBase> out(view(os, d->output, d->out_exponent, d->out_dtype));
    switch (d->op) {
    case ESPDL_ELT_ADD:
    case ESPDL_ELT_SUB:
    case ESPDL_ELT_MUL:
    case ESPDL_ELT_MAX:
    case ESPDL_ELT_MIN:
    case ESPDL_ELT_DIV:
    case ESPDL_ELT_MOD:
    case ESPDL_ELT_GREATER:
    case ESPDL_ELT_GREATER_EQUAL:
    case ESPDL_ELT_EQUAL:
    case ESPDL_ELT_LESS:
    case ESPDL_ELT_LESS_EQUAL:
    case ESPDL_ELT_POW: {
        std::unique_ptr<TensorBase> in1(view(s1, d->input1, d->in1_exponent, d->in_dtype));
        std::unique_ptr<module::Module> m;
        if (d->op == ESPDL_ELT_ADD)
            m.reset(new module::Add(nullptr, MODULE_NON_INPLACE, qt));
        else if (d->op == ESPDL_ELT_SUB)
            m.reset(new module::Sub(nullptr, MODULE_NON_INPLACE, qt));
        else if (d->op == ESPDL_ELT_MAX)
            m.reset(new module::Max(nullptr, MODULE_NON_INPLACE, qt));
        else if (d->op == ESPDL_ELT_MIN)
            m.reset(new module::Min(nullptr, MODULE_NON_INPLACE, qt));
        else if (d->op == ESPDL_ELT_DIV)
            m.reset(new module::Div(nullptr, MODULE_NON_INPLACE, qt));
        else if (d->op == ESPDL_ELT_MOD)
            m.reset(new module::Mod(nullptr, MODULE_NON_INPLACE, qt));
        else if (d->op == ESPDL_ELT_GREATER)
            m.reset(new module::Greater(nullptr, MODULE_NON_INPLACE, qt));
        else if (d->op == ESPDL_ELT_GREATER_EQUAL)
            m.reset(new module::GreaterOrEqual(nullptr, MODULE_NON_INPLACE, qt));
        else if (d->op == ESPDL_ELT_EQUAL)
            m.reset(new module::Equal(nullptr, MODULE_NON_INPLACE, qt));
        else if (d->op == ESPDL_ELT_LESS)
            m.reset(new module::Less(nullptr, MODULE_NON_INPLACE, qt));
        else if (d->op == ESPDL_ELT_LESS_EQUAL)
            m.reset(new module::LessOrEqual(nullptr, MODULE_NON_INPLACE, qt));
        else if (d->op == ESPDL_ELT_POW)
            m.reset(new module::Pow(nullptr, MODULE_NON_INPLACE, qt));
        else
            m.reset(new module::Mul(nullptr, MODULE_NON_INPLACE, qt));
        m->run({in0.get(), in1.get()}, {out.get()}, RUNTIME_MODE_SINGLE_CORE);
        return ESPDL_OK;
    }
    case ESPDL_ELT_REQUANTIZE: {
        module::RequantizeLinear m(nullptr, MODULE_NON_INPLACE, qt);
        m.run(in0.get(), out.get(), RUNTIME_MODE_SINGLE_CORE);
        return ESPDL_OK;
    }
    case ESPDL_ELT_LUT: {
        const int entries = d->in_dtype == ESPDL_DTYPE_INT16 ? (65536 >> d->lut_shift) + 1 : 256;
        TensorBase *table = new TensorBase({entries}, d->input1, d->out_exponent, to_dtype(d->in_dtype), true); /* owned by LUT */
        module::LUT m(nullptr, table, MODULE_NON_INPLACE, qt);
        m.run(in0.get(), out.get(), RUNTIME_MODE_SINGLE_CORE);
        return ESPDL_OK;
    }
    case ESPDL_ELT_CLIP: {
        /* min / max arrive as one-element tensors in the input's quantised scale */
        int16_t lo16 = (int16_t)d->clip_lo, hi16 = (int16_t)d->clip_hi;
        int8_t lo8 = (int8_t)d->clip_lo, hi8 = (int8_t)d->clip_hi;
        const void *lo = d->in_dtype == ESPDL_DTYPE_INT8 ? (const void *)&lo8 : (const void *)&lo16;
        const void *hi = d->in_dtype == ESPDL_DTYPE_INT8 ? (const void *)&hi8 : (const void *)&hi16;
        std::unique_ptr<TensorBase> tmin(new TensorBase({1}, lo, d->in0_exponent, to_dtype(d->in_dtype), true));
        std::unique_ptr<TensorBase> tmax(new TensorBase({1}, hi, d->in0_exponent, to_dtype(d->in_dtype), true));
        module::Clip m(nullptr, MODULE_NON_INPLACE, qt);
        m.run({in0.get(), tmin.get(), tmax.get()}, {out.get()}, RUNTIME_MODE_SINGLE_CORE);
        return ESPDL_OK;
    }
    case ESPDL_ELT_RELU: {
        module::Relu m(nullptr, MODULE_NON_INPLACE, qt);
        m.run(in0.get(), out.get(), RUNTIME_MODE_SINGLE_CORE);
        return ESPDL_OK;
    }
    case ESPDL_ELT_PRELU: {
        if (d->ndim != 4)
            return ESPDL_ERR_UNSUPPORTED;
        int c = d->out_shape[3];
        TensorBase *alpha = new TensorBase({c, 1, 1}, d->input1, d->in1_exponent, to_dtype(d->in_dtype), true); /* owned by PRelu */
        module::PRelu m(nullptr, alpha, MODULE_NON_INPLACE, qt);
        m.run(in0.get(), out.get(), RUNTIME_MODE_SINGLE_CORE);
        return ESPDL_OK;
    }
    default:
        return ESPDL_ERR_UNSUPPORTED;
    }
}

int ref_pool(const espdl_pool_desc *d)
{
    if (!d)
        return ESPDL_ERR_INVALID_ARG;
    const size_t es = esize(d->dtype);
    const quant_type_t qt = to_quant(d->dtype);
    const int oh = d->op == ESPDL_POOL_GLOBAL_AVG ? 1 : d->out_h, ow = d->op == ESPDL_POOL_GLOBAL_AVG ? 1 : d->out_w;
    for (int n = 0; n < d->n; n++) {
        const char *ip = (const char *)d->input + (size_t)n * d->in_h * d->in_w * d->c * es;
        char *op = (char *)d->output + (size_t)n * oh * ow * d->c * es;
        std::unique_ptr<TensorBase> in(view({1, d->in_h, d->in_w, d->c}, ip, d->in_exponent, d->dtype));
        std::unique_ptr<TensorBase> out(view({1, oh, ow, d->c}, op, d->out_exponent, d->dtype));
        std::vector<int> pads = {d->pad_top, d->pad_bottom, d->pad_left, d->pad_right};
        if (d->op == ESPDL_POOL_MAX) {
            module::MaxPool m(nullptr, {d->kh, d->kw}, pads, {d->stride_h, d->stride_w}, qt);
            m.run(in.get(), out.get(), RUNTIME_MODE_SINGLE_CORE);
        } else if (d->op == ESPDL_POOL_AVG) {
            module::AveragePool m(nullptr, {d->kh, d->kw}, pads, {d->stride_h, d->stride_w}, qt);
            m.run(in.get(), out.get(), RUNTIME_MODE_SINGLE_CORE);
        } else {
            module::GlobalAveragePool m(nullptr, qt);
            m.run(in.get(), out.get(), RUNTIME_MODE_SINGLE_CORE);
        }
    }
    return ESPDL_OK;
}

int ref_resize(const espdl_resize_desc *d)
{
    if (!d || (d->out_pixel_stride && d->out_pixel_stride != d->c))
        return ESPDL_ERR_UNSUPPORTED;
    const size_t es = esize(d->dtype);
    for (int n = 0; n < d->n; n++) {
        const char *ip = (const char *)d->input + (size_t)n * d->in_h * d->in_w * d->c * es;
        char *op = (char *)d->output + (size_t)n * d->out_h * d->out_w * d->c * es;
        if (d->mode != 0 && d->in_h == 1 && d->out_h == 1) { // linear along w: the reference's 3-D (NWC) form
            std::unique_ptr<TensorBase> in(view({1, d->in_w, d->c}, ip, d->in_exponent, d->dtype));
            std::unique_ptr<TensorBase> out(view({1, d->out_w, d->c}, op, d->out_exponent, d->dtype));
            module::Resize m(nullptr, RESIZE_LINEAR, {1.f, 1.f, d->scale_w}, {}, d->mode == 2, to_quant(d->dtype));
            m.run(in.get(), out.get(), RUNTIME_MODE_SINGLE_CORE);
            continue;
        }
        std::unique_ptr<TensorBase> in(view({1, d->in_h, d->in_w, d->c}, ip, d->in_exponent, d->dtype));
        std::unique_ptr<TensorBase> out(view({1, d->out_h, d->out_w, d->c}, op, d->out_exponent, d->dtype));
        module::Resize m(nullptr, d->mode == 0 ? RESIZE_NEAREST : RESIZE_LINEAR, {1.f, 1.f, d->scale_h, d->scale_w}, {}, d->mode == 2,
                         to_quant(d->dtype));
        m.run(in.get(), out.get(), RUNTIME_MODE_SINGLE_CORE);
    }
    return ESPDL_OK;
}

/* Softmax over the last axis of an int8 [rows, len] tensor into float32. */
int ref_softmax(const espdl_softmax_desc *d, int in_exponent)
{
    if (!d || d->out_dtype != ESPDL_DTYPE_FLOAT)
        return ESPDL_ERR_UNSUPPORTED;
    if (d->log) { /* LogSoftmax along axis 1 of [outer, len, inner] */
        const int inner = d->inner > 1 ? d->inner : 1;
        std::vector<int> shape = {d->rows / inner, d->len, inner};
        if (inner == 1)
            shape.pop_back();
        std::unique_ptr<TensorBase> in(view(shape, d->input, in_exponent, ESPDL_DTYPE_INT8));
        std::unique_ptr<TensorBase> out(view(shape, d->output, 0, ESPDL_DTYPE_FLOAT));
        module::LogSoftmax m(nullptr, 1, MODULE_NON_INPLACE, QUANT_TYPE_SYMM_8BIT);
        m.run(in.get(), out.get(), RUNTIME_MODE_SINGLE_CORE);
        return ESPDL_OK;
    }
    std::unique_ptr<TensorBase> in(view({d->rows, d->len}, d->input, in_exponent, ESPDL_DTYPE_INT8));
    std::unique_ptr<TensorBase> out(view({d->rows, d->len}, d->output, 0, ESPDL_DTYPE_FLOAT));
    module::Softmax m(nullptr, -1, MODULE_NON_INPLACE, QUANT_TYPE_SYMM_8BIT);
    m.run(in.get(), out.get(), RUNTIME_MODE_SINGLE_CORE);
    return ESPDL_OK;
}

/* Concat of two int8 tensors along `axis` (checks the copy descriptors the backend derives). */
int ref_concat2(const int8_t *a, const int8_t *b, int8_t *out, const int *shape_a, const int *shape_b, int ndim, int axis)
{
    std::vector<int> sa(shape_a, shape_a + ndim), sb(shape_b, shape_b + ndim), so(sa);
    so[axis] += sb[axis];
    std::unique_ptr<TensorBase> ta(view(sa, a, 0, ESPDL_DTYPE_INT8)), tb(view(sb, b, 0, ESPDL_DTYPE_INT8)),
        to(view(so, out, 0, ESPDL_DTYPE_INT8));
    module::Concat m(nullptr, axis, QUANT_TYPE_SYMM_8BIT);
    std::vector<std::vector<int>> shapes = {sa, sb};
    m.get_output_shape(shapes);
    m.run({ta.get(), tb.get()}, {to.get()}, RUNTIME_MODE_SINGLE_CORE);
    return ESPDL_OK;
}

/* MatMul through the reference's own module (dl_module_matmul.hpp:125-526): shapes of up to four dims with its
 * broadcasting rules, per-tensor exponents, no bias. */
int ref_matmul(const void *a, const int *shape_a, int ndim_a, int e_a, const void *b, const int *shape_b, int ndim_b, int e_b, void *out,
               int e_out, int dtype, int relu)
{
    std::vector<int> sa(shape_a, shape_a + ndim_a), sb(shape_b, shape_b + ndim_b);
    module::MatMul m(relu ? ReLU : Linear, "matmul", to_quant(dtype));
    std::vector<std::vector<int>> in_shapes = {sa, sb};
    std::vector<int> so = m.get_output_shape(in_shapes)[0];
    std::unique_ptr<TensorBase> ta(view(sa, a, e_a, dtype)), tb(view(sb, b, e_b, dtype)), to(view(so, out, e_out, dtype));
    m.run({ta.get(), tb.get()}, {to.get()}, RUNTIME_MODE_SINGLE_CORE);
    return 0;
}

/* ReduceMean / ReduceSum / ReduceMax / ReduceMin through the reference's own modules (dl_module_reduce_*.hpp). */
int ref_reduce(const espdl_reduce_desc *d)
{
    std::vector<int> shape(d->shape, d->shape + d->ndim);
    std::vector<bool> flags;
    for (int i = 0; i < d->ndim; i++) flags.push_back(d->reduce[i] != 0);
    std::unique_ptr<module::Module> m;
    const quant_type_t q = to_quant(d->dtype);
    if (d->op == ESPDL_REDUCE_MEAN)
        m.reset(new module::ReduceMean(1, flags, "ReduceMean", "reduce", MODULE_NON_INPLACE, q));
    else if (d->op == ESPDL_REDUCE_SUM)
        m.reset(new module::ReduceSum(1, flags, "ReduceSum", "reduce", MODULE_NON_INPLACE, q));
    else if (d->op == ESPDL_REDUCE_MAX)
        m.reset(new module::ReduceMax(1, flags, "ReduceMax", "reduce", MODULE_NON_INPLACE, q));
    else if (d->op == ESPDL_REDUCE_L1)
        m.reset(new module::ReduceL1(1, flags, "ReduceL1", "reduce", MODULE_NON_INPLACE, q));
    else if (d->op == ESPDL_REDUCE_SUM_SQUARE)
        m.reset(new module::ReduceSumSquare(1, flags, "ReduceSumSquare", "reduce", MODULE_NON_INPLACE, q));
    else if (d->op == ESPDL_REDUCE_L2)
        m.reset(new module::ReduceL2(1, flags, "ReduceL2", "reduce", MODULE_NON_INPLACE, q));
    else if (d->op == ESPDL_REDUCE_PROD)
        m.reset(new module::ReduceProd(1, flags, "ReduceProd", "reduce", MODULE_NON_INPLACE, q));
    else if (d->op == ESPDL_REDUCE_LOG_SUM)
        m.reset(new module::ReduceLogSum(1, flags, "ReduceLogSum", "reduce", MODULE_NON_INPLACE, q));
    else if (d->op == ESPDL_REDUCE_LOG_SUM_EXP)
        m.reset(new module::ReduceLogSumExp(1, flags, "ReduceLogSumExp", "reduce", MODULE_NON_INPLACE, q));
    else
        m.reset(new module::ReduceMin(1, flags, "ReduceMin", "reduce", MODULE_NON_INPLACE, q));
    std::vector<std::vector<int>> in_shapes = {shape};
    std::vector<int> so = m->get_output_shape(in_shapes)[0];
    std::unique_ptr<TensorBase> ti(view(shape, d->input, d->in_exponent, d->dtype)), to(view(so, d->output, d->out_exponent, d->dtype));
    m->run({ti.get()}, {to.get()}, RUNTIME_MODE_SINGLE_CORE);
    return 0;
}

/* Gather through the reference's own module; `shape` is the input shape, the indices are a 1-D int32 tensor. */
int ref_gather(const void *input, void *output, const int32_t *indices, int num_indices, const int *shape, int ndim, int axis, int dtype)
{
    std::vector<int> sh(shape, shape + ndim);
    module::Gather m(new TensorBase({num_indices}, indices, 0, DATA_TYPE_INT32, true), axis, "gather", MODULE_NON_INPLACE, to_quant(dtype));
    std::vector<std::vector<int>> in_shapes = {sh};
    std::vector<int> so = m.get_output_shape(in_shapes)[0];
    std::unique_ptr<TensorBase> ti(view(sh, input, 0, dtype)), to(view(so, output, 0, dtype));
    m.run({ti.get()}, {to.get()}, RUNTIME_MODE_SINGLE_CORE);
    return 0;
}

/* mode 0 SpaceToDepth, 1 DepthToSpace "DCR", 2 DepthToSpace "CRD" through the reference's own modules (NHWC input extents). */
int ref_depth_space(const void *input, void *output, int dtype, int n, int h, int w, int c, int bs, int mode)
{
    std::unique_ptr<module::Module> m;
    if (mode == 0)
        m.reset(new module::SpaceToDepth(bs, "s2d", MODULE_NON_INPLACE, to_quant(dtype)));
    else
        m.reset(new module::DepthToSpace(bs, mode == 1 ? "DCR" : "CRD", "d2s", MODULE_NON_INPLACE, to_quant(dtype)));
    std::vector<int> sh = {n, h, w, c};
    std::vector<std::vector<int>> in_shapes = {sh};
    std::vector<int> so = m->get_output_shape(in_shapes)[0];
    std::unique_ptr<TensorBase> ti(view(sh, input, 0, dtype)), to(view(so, output, 0, dtype));
    m->run({ti.get()}, {to.get()}, RUNTIME_MODE_SINGLE_CORE);
    return 0;
}

/* RMSNormalization / LayerNormalization through the reference's own modules (rows x len, normalised over the last axis). */
int ref_norm(const espdl_norm_desc *d)
{
    const int rows = (int)d->rows, len = d->len;
    std::vector<std::unique_ptr<TensorBase>> keep;
    auto mk = [&](std::vector<int> shape, const void *p, int e, int dtype) {
        keep.emplace_back(view(shape, p, e, dtype));
        return keep.back().get();
    };
    std::vector<TensorBase *> ins = {mk({rows, len}, d->input, d->in_exponent, d->dtype)}, outs;
    std::unique_ptr<module::Module> m;
    if (d->op == ESPDL_NORM_RMS) {
        ins.push_back(mk({len}, d->scale, 0, ESPDL_DTYPE_FLOAT));
        m.reset(new module::RMSNormalization(-1, d->epsilon, "rms", MODULE_NON_INPLACE, to_quant(d->dtype)));
    } else {
        if (d->scale)
            ins.push_back(mk({len}, d->scale, d->scale_exponent, d->dtype));
        if (d->scale && d->bias)
            ins.push_back(mk({len}, d->bias, d->bias_exponent, d->dtype));
        m.reset(new module::LayerNormalization(-1, d->epsilon, 1, "ln", MODULE_NON_INPLACE, to_quant(d->dtype)));
    }
    outs.push_back(mk({rows, len}, d->output, d->out_exponent, d->dtype));
    if (d->op == ESPDL_NORM_LAYER && d->mean && d->inv_std_dev) {
        outs.push_back(mk({rows, 1}, d->mean, d->mean_exponent, d->dtype));
        outs.push_back(mk({rows, 1}, d->inv_std_dev, d->inv_std_dev_exponent, d->dtype));
    }
    m->run(ins, outs, RUNTIME_MODE_SINGLE_CORE);
    return 0;
}

/* InsertZeros through the reference's own module: NWC / NHWC input of `ndim` axes, one stride and padding per spatial axis. */
int ref_insert_zeros(const void *input, void *output, int dtype, const int *shape, int ndim, const int *stride, const int *output_padding)
{
    std::vector<int> sh(shape, shape + ndim), st(stride, stride + ndim - 2), op(output_padding, output_padding + ndim - 2);
    module::InsertZeros m("iz", st, op, to_quant(dtype));
    std::vector<std::vector<int>> in_shapes = {sh};
    std::vector<int> so = m.get_output_shape(in_shapes)[0];
    std::unique_ptr<TensorBase> ti(view(sh, input, 0, dtype)), to(view(so, output, 0, dtype));
    m.run(ti.get(), to.get(), RUNTIME_MODE_SINGLE_CORE);
    return 0;
}

/* Pad through the reference's own module (dl_module_pad.hpp): int8 / int16 tensors. */
int ref_pad(const espdl_pad_desc *d)
{
    std::vector<int> shape(d->shape, d->shape + d->ndim), pads;
    for (int i = 0; i < d->ndim; i++) pads.push_back(d->pad_begin[i]);
    for (int i = 0; i < d->ndim; i++) pads.push_back(d->pad_end[i]);
    const int dtype = d->elem_size == 1 ? ESPDL_DTYPE_INT8 : ESPDL_DTYPE_INT16;
    const padding_mode_t mode = d->mode == ESPDL_PAD_CONSTANT ? PADDING_CONSTANT : (d->mode == ESPDL_PAD_EDGE ? PADDING_EDGE : PADDING_REFLECT);
    int8_t c8 = (int8_t)d->constant;
    int16_t c16 = (int16_t)d->constant;
    TensorBase *cv = view({1}, d->elem_size == 1 ? (const void *)&c8 : (const void *)&c16, 0, dtype);
    module::Pad m(pads, mode, new TensorBase({1}, cv->data, 0, cv->dtype, true), "pad", MODULE_NON_INPLACE, to_quant(dtype));
    delete cv;
    std::vector<std::vector<int>> in_shapes = {shape};
    std::vector<int> so = m.get_output_shape(in_shapes)[0];
    std::unique_ptr<TensorBase> ti(view(shape, d->input, 0, dtype)), to(view(so, d->output, 0, dtype));
    m.run({ti.get()}, {to.get()}, RUNTIME_MODE_SINGLE_CORE);
    return 0;
}

/* The reference's own YOLO11 post-processor (esp-dl/vision/detect/dl_detect_yolo11_postprocessor.cpp:8-96 over
 * dl_detect_postprocessor.cpp:5-50), unmodified, on host tensors: three (or fewer) heads named score<i> / box<i>.
 * Same arguments and result layout as oracle_yolo11_postprocess: boxes[5*i] = category, then the clipped box; returns
 * the number of results. */
struct ref_det_stage {
    const int8_t *score, *box;
    int h, w, classes, score_exponent, box_exponent, stride_y, stride_x, offset_y, offset_x;
};

int ref_yolo11_postprocess(const ref_det_stage *stages, int n_stages, float score_thr, float nms_thr, int top_k, float inv_scale_x,
                           float inv_scale_y, int border_left, int border_top, int width, int height, int round_mode, int max_results,
                           int *boxes, float *scores)
{
    (void)round_mode; /* the host build rounds half up, as every generic-C build of the reference does */
    if (n_stages != 3)
        return -1; /* postprocess() reads exactly score0..2 / box0..2 */
    dl::Model model;
    dl::image::ImagePreprocessor pre;
    pre.inv_scale_x = inv_scale_x, pre.inv_scale_y = inv_scale_y, pre.border_left = border_left, pre.border_top = border_top;
    std::vector<dl::TensorBase *> owned;
    std::vector<dl::detect::anchor_point_stage_t> geo;
    for (int i = 0; i < n_stages; i++) {
        const ref_det_stage &st = stages[i];
        dl::TensorBase *sc = new dl::TensorBase({1, st.h, st.w, st.classes}, st.score, st.score_exponent, dl::DATA_TYPE_INT8, false);
        dl::TensorBase *bx = new dl::TensorBase({1, st.h, st.w, 64}, st.box, st.box_exponent, dl::DATA_TYPE_INT8, false);
        owned.push_back(sc), owned.push_back(bx);
        model.outputs["score" + std::to_string(i)] = sc;
        model.outputs["box" + std::to_string(i)] = bx;
        geo.push_back({st.stride_y, st.stride_x, st.offset_y, st.offset_x});
    }
    dl::detect::yolo11PostProcessor post(&model, &pre, score_thr, nms_thr, top_k, geo);
    post.postprocess();
    std::list<dl::detect::result_t> &res = post.get_result(width, height);
    int n = 0;
    for (const dl::detect::result_t &r : res) {
        if (n >= max_results)
            break;
        boxes[5 * n] = r.category;
        for (int j = 0; j < 4; j++) boxes[5 * n + 1 + j] = r.box[j];
        scores[n] = r.score;
        n++;
    }
    for (dl::TensorBase *t : owned) delete t;
    return n;
}

/* The reference's NormQuant tables (esp-dl/vision/image/dl_image_norm_quant.hpp:13-31), three channels, int8 or int16:
 * `table` receives 3 * 256 entries. */
int ref_norm_quant_table(void *table, const float *mean, const float *std, int exponent, int bits)
{
    const std::array<float, 3> m = {mean[0], mean[1], mean[2]}, s = {std[0], std[1], std[2]};
    if (bits == 8) {
        dl::image::NormQuant<int8_t, 3> nq(m, s, exponent);
        memcpy(table, nq.m_lut1, 3 * 256);
    } else if (bits == 16) {
        dl::image::NormQuant<int16_t, 3> nq(m, s, exponent);
        memcpy(table, nq.m_lut1, 3 * 256 * 2);
    } else {
        return -1;
    }
    return 0;
}


/* LpNormalization along axis 1 of [outer, len, inner] (inner == 1: the last axis of [outer, len]). */
int ref_lp_norm(const espdl_norm_desc *d)
{
    const int inner = d->inner > 1 ? (int)d->inner : 1;
    std::vector<int> shape = {(int)(d->rows / inner), d->len, inner};
    if (inner == 1)
        shape.pop_back();
    std::unique_ptr<TensorBase> in(view(shape, d->input, d->in_exponent, d->dtype)), out(view(shape, d->output, d->out_exponent, d->dtype));
    module::LpNormalization m(1, d->p, nullptr, MODULE_NON_INPLACE, to_quant(d->dtype));
    m.run(in.get(), out.get(), RUNTIME_MODE_SINGLE_CORE);
    return 0;
}

/* ReverseSequence: input [dim0, dim1, feature], seq_lens int64[batch] on the host. */
int ref_reverse_sequence(const espdl_reverse_sequence_desc *d, const int64_t *seq_lens)
{
    const int batch = d->batch_axis == 0 ? d->dim0 : d->dim1;
    std::vector<int> shape = {d->dim0, d->dim1, (int)d->feature};
    const int dt = d->elem_size == 1 ? ESPDL_DTYPE_INT8 : (d->elem_size == 2 ? ESPDL_DTYPE_INT16 : ESPDL_DTYPE_FLOAT);
    std::unique_ptr<TensorBase> in(view(shape, d->input, 0, dt)), out(view(shape, d->output, 0, dt));
    std::unique_ptr<TensorBase> lens(view({batch}, seq_lens, 0, ESPDL_DTYPE_INT64));
    module::ReverseSequence m(d->batch_axis, 1 - d->batch_axis, nullptr, MODULE_NON_INPLACE, to_quant(dt));
    m.run({in.get(), lens.get()}, {out.get()}, RUNTIME_MODE_SINGLE_CORE);
    return 0;
}

/* ScatterND: data of shape `shape`, indices [n_slices, index_depth] int64, updates [n_slices, slice dims...]. */
int ref_scatter_nd(const espdl_scatter_nd_desc *d, const int *shape, int ndim)
{
    static const char *names[] = {"none", "add", "mul", "max", "min"};
    std::vector<int> ds(shape, shape + ndim), is = {d->n_slices, d->index_depth}, us = {d->n_slices};
    for (int i = d->index_depth; i < ndim; i++) us.push_back(shape[i]);
    std::unique_ptr<TensorBase> data(view(ds, d->data, 0, d->dtype)), out(view(ds, d->output, 0, d->dtype));
    std::unique_ptr<TensorBase> idx(view(is, d->indices, 0, ESPDL_DTYPE_INT64)), upd(view(us, d->updates, 0, d->dtype));
    module::ScatterND m(names[d->reduction], nullptr, MODULE_NON_INPLACE, to_quant(d->dtype));
    m.run({data.get(), idx.get(), upd.get()}, {out.get()}, RUNTIME_MODE_SINGLE_CORE);
    return 0;
}

/* GRU / LSTM through the reference's own modules: inputs X, W, R, B, (sequence_lens, unused), initial_h, initial_c in the
 * operator's input order; absent optional inputs end the list (an absent B with a present initial_h cannot be expressed
 * by position and is not pinned). */
int ref_rnn(const espdl_rnn_desc *d)
{
    const int H = d->hidden_size, G = d->op == ESPDL_RNN_GRU ? 3 : 4, D = d->directions;
    std::unique_ptr<TensorBase> x(view({d->seq_length, 1, d->input_size}, d->x, d->x_exponent, d->dtype));
    std::unique_ptr<TensorBase> w(view({D, G * H, d->input_size}, d->w, d->w_exponent, d->dtype));
    std::unique_ptr<TensorBase> r(view({D, G * H, H}, d->r, d->r_exponent, d->dtype));
    std::unique_ptr<TensorBase> b, lens, h0, c0;
    int64_t seq_lens[1] = {d->seq_length};
    std::vector<TensorBase *> ins = {x.get(), w.get(), r.get()};
    if (d->b) {
        b.reset(view({D, 2 * G * H}, d->b, d->gate_exponent, ESPDL_DTYPE_INT16));
        ins.push_back(b.get());
        if (d->initial_h) {
            lens.reset(view({1}, seq_lens, 0, ESPDL_DTYPE_INT64));
            h0.reset(view({D, 1, H}, d->initial_h, d->h_exponent, d->dtype));
            ins.push_back(lens.get());
            ins.push_back(h0.get());
            if (d->op == ESPDL_RNN_LSTM && d->initial_c) {
                c0.reset(view({D, 1, H}, d->initial_c, d->gate_exponent, ESPDL_DTYPE_INT16));
                ins.push_back(c0.get());
            }
        }
    } else if (d->initial_h) {
        return ESPDL_ERR_UNSUPPORTED;
    }
    std::unique_ptr<TensorBase> y(view({d->seq_length, D, 1, H}, d->y, d->y_exponent, d->dtype));
    std::unique_ptr<TensorBase> yh(view({D, 1, H}, d->y_h, d->h_exponent, d->dtype));
    if (d->op == ESPDL_RNN_GRU) {
        module::GRU m(nullptr, H, D, 0, d->gate_exponent, MODULE_NON_INPLACE, to_quant(d->dtype));
        m.run(ins, {y.get(), yh.get()}, RUNTIME_MODE_SINGLE_CORE);
    } else {
        std::unique_ptr<TensorBase> yc(view({D, 1, H}, d->y_c, d->c_exponent, ESPDL_DTYPE_INT16));
        module::LSTM m(nullptr, H, D, 0, d->gate_exponent, MODULE_NON_INPLACE, to_quant(d->dtype));
        m.run(ins, {y.get(), yh.get(), yc.get()}, RUNTIME_MODE_SINGLE_CORE);
    }
    return 0;
}
} /* extern "C" */
