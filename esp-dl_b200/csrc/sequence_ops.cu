// LpNormalization, ReverseSequence and ScatterND: the operators of ESP-DL's list whose arithmetic is a walk over one
// axis or over index tuples.  Replaces dl::module::LpNormalization::forward_int8 / forward_int16
// (esp-dl/dl/module/include/dl_module_lp_normalization.hpp:122-262, 300-356), dl::module::ReverseSequence
// (dl_module_reverse_sequence.hpp:14-58) and dl::module::ScatterND::forward_template (dl_module_scatter_nd.hpp:160-228).
#include "common.cuh"

namespace espdl {

namespace {

// ------------------------------------------------------------------------------------------ LpNormalization
// One thread per row (one position of the other axes).  p = 2: the sum of squares is an integer (exact in any order),
// 1 / sqrtf of it and every product are correctly rounded single operations, so the result is the reference's bit for
// bit.  p = 1: the reference adds |x| as floats in element order; so does the thread.  The reference multiplies in two
// different orders: along the last axis y = round(x * (inv_norm * 2^-e_out)), along any other axis
// y = round((x * inv_norm) * 2^-e_out).
template <typename T>
__global__ void __launch_bounds__(128) lp_norm_kernel(const T *in, T *out, long long rows, int len, long long inner, int p, float out_rescale, int half_even)
{
    for (long long r = blockIdx.x * (long long)blockDim.x + threadIdx.x; r < rows; r += (long long)gridDim.x * blockDim.x) {
        const long long base = (r / inner) * (long long)len * inner + (r % inner);
        float inv_norm;
        if (p == 1) {
            float sum_abs = 0.f;
            for (int i = 0; i < len; i++) sum_abs = __fadd_rn(sum_abs, fabsf((float)(int)in[base + i * inner]));
            inv_norm = sum_abs > 0.f ? __fdiv_rn(1.f, sum_abs) : 0.f;
        } else {
            long long sq = 0;
            for (int i = 0; i < len; i++) {
                const long long v = in[base + i * inner];
                sq += v * v;
            }
            // reduce_l2 returns int32 for int8 and int64 for int16 (dl_base_reduce.cpp:11-110); then static_cast<float>
            const float sum_sq = sizeof(T) == 1 ? __int2float_rn((int)sq) : __ll2float_rn(sq);
            inv_norm = sum_sq > 0.f ? __fdiv_rn(1.f, __fsqrt_rn(sum_sq)) : 0.f; // math::fast_inv_sqrt without DL_FAST_MATH
        }
        const bool last_axis = inner == 1;
        const float scaled = __fmul_rn(inv_norm, out_rescale);
        const bool live = last_axis ? scaled > 0.f : inv_norm > 0.f;
        for (int i = 0; i < len; i++) {
            int q = 0;
            if (live) {
                const float x = (float)(int)in[base + i * inner];
                q = last_axis ? fround(__fmul_rn(x, scaled), half_even) : fround(__fmul_rn(__fmul_rn(x, inv_norm), out_rescale), half_even);
            }
            out[base + i * inner] = (T)(sizeof(T) == 1 ? sat8(q) : sat16(q));
        }
    }
}

// ------------------------------------------------------------------------------------------ ReverseSequence
template <typename T>
__global__ void __launch_bounds__(256) reverse_sequence_kernel(const T *in, T *out, const long long *seq_lens, int batch_axis, int dim0, int dim1,
                                                               long long feature, long long total)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long f = i % feature;
        const long long r = i / feature;
        const int i1 = (int)(r % dim1), i0 = (int)(r / dim1);
        const int b = batch_axis == 0 ? i0 : i1, t = batch_axis == 0 ? i1 : i0;
        const long long len = seq_lens[b];
        const int time = batch_axis == 0 ? dim1 : dim0;
        // the reference swaps steps t and len-1-t for t < len/2 in place; a length beyond the axis is the caller's error
        int ts = t;
        if (len > 1 && len <= time && t < len)
            ts = (int)(len - 1 - t);
        const long long src = batch_axis == 0 ? ((long long)i0 * dim1 + ts) * feature + f : ((long long)ts * dim1 + i1) * feature + f;
        out[i] = in[src];
    }
}

// ------------------------------------------------------------------------------------------ ScatterND
// Slices are visited in order by every thread; a thread owns one position inside the slice, so two updates of the same
// output element are applied by the same thread in the reference's order (slices are identical or disjoint because an
// index tuple addresses whole slices).
template <typename T>
__device__ __forceinline__ T scatter_apply(T cur, T upd, int reduction)
{
    if (reduction == ESPDL_SCATTER_NONE)
        return upd;
    if (reduction == ESPDL_SCATTER_MAX)
        return cur > upd ? cur : upd;
    if (reduction == ESPDL_SCATTER_MIN)
        return cur < upd ? cur : upd;
    if (sizeof(T) == 4) { // float
        return reduction == ESPDL_SCATTER_ADD ? (T)__fadd_rn((float)cur, (float)upd) : (T)__fmul_rn((float)cur, (float)upd);
    }
    const int lo = sizeof(T) == 1 ? -128 : -32768, hi = sizeof(T) == 1 ? 127 : 32767;
    const int v = reduction == ESPDL_SCATTER_ADD ? (int)cur + (int)upd : (int)cur * (int)upd;
    return (T)max(lo, min(hi, v));
}

template <typename T>
__global__ void __launch_bounds__(256) scatter_nd_kernel(espdl_scatter_nd_desc d)
{
    T *out = (T *)d.output;
    const T *upd = (const T *)d.updates;
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < d.slice_size; e += (long long)gridDim.x * blockDim.x) {
        for (int s = 0; s < d.n_slices; s++) {
            long long flat = 0;
            for (int k = 0; k < d.index_depth; k++) flat += d.indices[(long long)s * d.index_depth + k] * d.axis_offset[k];
            if (flat < 0 || flat + d.slice_size > d.data_size)
                continue; // an index outside the tensor: the reference writes outside its buffer, this kernel skips it
            out[flat + e] = scatter_apply<T>(out[flat + e], upd[(long long)s * d.slice_size + e], d.reduction);
        }
    }
}

} // namespace

int lp_norm_op(const espdl_norm_desc &d, cudaStream_t s)
{
    if ((d.p != 1 && d.p != 2) || d.inner < 1 || d.rows % d.inner != 0)
        return ESPDL_ERR_INVALID_ARG;
    const long long blocks = (d.rows + 127) / 128;
    const unsigned grid = (unsigned)min(blocks, (long long)num_sms() * 16);
    const int he = d.round_mode == ESPDL_ROUND_HALF_EVEN;
    if (d.dtype == ESPDL_DTYPE_INT8)
        lp_norm_kernel<int8_t><<<grid, 128, 0, s>>>((const int8_t *)d.input, (int8_t *)d.output, d.rows, d.len, d.inner, d.p, dl_rescale(d.out_exponent), he);
    else
        lp_norm_kernel<int16_t><<<grid, 128, 0, s>>>((const int16_t *)d.input, (int16_t *)d.output, d.rows, d.len, d.inner, d.p, dl_rescale(d.out_exponent), he);
    count_launch();
    return check_launch("lp_norm");
}

} // namespace espdl

using namespace espdl;

extern "C" int espdl_b200_reverse_sequence(const espdl_reverse_sequence_desc *d, void *stream)
{
    if (!d || !d->input || !d->output || !d->seq_lens || d->input == d->output || d->dim0 <= 0 || d->dim1 <= 0 || d->feature <= 0 ||
        (d->batch_axis != 0 && d->batch_axis != 1))
        return ESPDL_ERR_INVALID_ARG;
    if (d->elem_size != 1 && d->elem_size != 2 && d->elem_size != 4)
        return ESPDL_ERR_UNSUPPORTED;
    const long long total = (long long)d->dim0 * d->dim1 * d->feature;
    const unsigned grid = (unsigned)min((total + 255) / 256, (long long)num_sms() * 16);
    cudaStream_t s = (cudaStream_t)stream;
    const long long *lens = (const long long *)d->seq_lens;
    if (d->elem_size == 1)
        reverse_sequence_kernel<int8_t><<<grid, 256, 0, s>>>((const int8_t *)d->input, (int8_t *)d->output, lens, d->batch_axis, d->dim0, d->dim1, d->feature, total);
    else if (d->elem_size == 2)
        reverse_sequence_kernel<int16_t><<<grid, 256, 0, s>>>((const int16_t *)d->input, (int16_t *)d->output, lens, d->batch_axis, d->dim0, d->dim1, d->feature, total);
    else
        reverse_sequence_kernel<int32_t><<<grid, 256, 0, s>>>((const int32_t *)d->input, (int32_t *)d->output, lens, d->batch_axis, d->dim0, d->dim1, d->feature, total);
    count_launch();
    return check_launch("reverse_sequence");
}

extern "C" int espdl_b200_scatter_nd(const espdl_scatter_nd_desc *d, void *stream)
{
    if (!d || !d->data || !d->output || d->n_slices < 0 || d->index_depth < 1 || d->index_depth > 6 || d->slice_size < 1 || d->data_size < 1 ||
        d->reduction < ESPDL_SCATTER_NONE || d->reduction > ESPDL_SCATTER_MIN)
        return ESPDL_ERR_INVALID_ARG;
    if (d->n_slices > 0 && (!d->indices || !d->updates))
        return ESPDL_ERR_INVALID_ARG;
    if (d->dtype != ESPDL_DTYPE_INT8 && d->dtype != ESPDL_DTYPE_INT16 && d->dtype != ESPDL_DTYPE_FLOAT)
        return ESPDL_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t es = d->dtype == ESPDL_DTYPE_INT8 ? 1 : (d->dtype == ESPDL_DTYPE_INT16 ? 2 : 4);
    if (d->data != d->output)
        ESPDL_CUDA_TRY(cudaMemcpyAsync(d->output, d->data, (size_t)d->data_size * es, cudaMemcpyDeviceToDevice, s));
    if (d->n_slices == 0)
        return ESPDL_OK;
    const unsigned grid = (unsigned)min((long long)((d->slice_size + 255) / 256), (long long)num_sms() * 8);
    if (d->dtype == ESPDL_DTYPE_INT8)
        scatter_nd_kernel<int8_t><<<grid, 256, 0, s>>>(*d);
    else if (d->dtype == ESPDL_DTYPE_INT16)
        scatter_nd_kernel<int16_t><<<grid, 256, 0, s>>>(*d);
    else
        scatter_nd_kernel<float><<<grid, 256, 0, s>>>(*d);
    count_launch();
    return check_launch("scatter_nd");
}
