// int8 Softmax along the last axis through the reference's 256-entry exp table
// (esp-dl/dl/module/include/dl_module_softmax.hpp:148-187).  The reference adds the row's
// exponentials sequentially in fp32, and fp32 addition is not associative, so a parallel
// reduction would change low bits: each row's sum is formed by ONE thread in index order,
// from a shared-memory copy of the row; the normalising divisions then run across the block.
// out_dtype INT8/INT16 folds in the QuantizeLinear node that follows it in exported graphs
// (esp-dl/dl/tensor/src/dl_tensor_base.cpp:251-264).  The softmax axis may be any axis: a "row" is the `len` elements
// that lie `inner` apart.  LogSoftmax on int8 (dl_module_log_softmax.hpp:150-215) uses the same table and the same
// sequential sum: y = 2^e_in * x - logf(sum), with logf evaluated on the device.
#include "common.cuh"

namespace espdl {

__global__ void __launch_bounds__(128) softmax_kernel(espdl_softmax_desc d, float out_rescale)
{
    __shared__ float table[256];
    __shared__ float sum_s;
    extern __shared__ int8_t row[];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) table[i] = d.exp_table[i];
    const int inner = d.inner > 1 ? d.inner : 1;
    const float in_scale = dl_scale(d.in_exponent);
    for (int r = blockIdx.x; r < d.rows; r += gridDim.x) {
        __syncthreads();
        const long long base = (long long)(r / inner) * d.len * inner + (r % inner);
        const int8_t *x = d.input + base;
        for (int i = threadIdx.x; i < d.len; i += blockDim.x) row[i] = x[(long long)i * inner];
        __syncthreads();
        if (threadIdx.x == 0) {
            float sum = 0.f;
            for (int i = 0; i < d.len; i++) sum = __fadd_rn(sum, table[row[i] + 128]);
            sum_s = d.log ? logf(sum) : sum;
        }
        __syncthreads();
        const float sum = sum_s;
        for (int i = threadIdx.x; i < d.len; i += blockDim.x) {
            const float y = d.log ? __fsub_rn(__fmul_rn(in_scale, (float)row[i]), sum) : __fdiv_rn(table[row[i] + 128], sum);
            const long long oi = base + (long long)i * inner;
            if (d.out_dtype == ESPDL_DTYPE_FLOAT)
                ((float *)d.output)[oi] = y;
            else if (d.out_dtype == ESPDL_DTYPE_INT8)
                ((int8_t *)d.output)[oi] = (int8_t)sat8(fround_half_up(__fmul_rn(y, out_rescale)));
            else
                ((int16_t *)d.output)[oi] = (int16_t)sat16(fround_half_up(__fmul_rn(y, out_rescale)));
        }
    }
}

} // namespace espdl

using namespace espdl;

extern "C" int espdl_b200_softmax(const espdl_softmax_desc *d, void *stream)
{
    if (!d || !d->input || !d->output || !d->exp_table || d->rows < 0 || d->len <= 0)
        return ESPDL_ERR_INVALID_ARG;
    if (d->out_dtype != ESPDL_DTYPE_FLOAT && d->out_dtype != ESPDL_DTYPE_INT8 && d->out_dtype != ESPDL_DTYPE_INT16)
        return ESPDL_ERR_UNSUPPORTED;
    if (d->len > 48 * 1024)
        return ESPDL_ERR_TOO_LARGE;
    if (d->out_exponent > 30 || d->out_exponent < -30 || d->in_exponent > 30 || d->in_exponent < -30 || d->inner < 0)
        return ESPDL_ERR_INVALID_ARG;
    if (d->inner > 1 && d->rows % d->inner != 0)
        return ESPDL_ERR_INVALID_ARG;
    if (d->rows == 0)
        return ESPDL_OK;
    const int blocks = min(d->rows, num_sms() * 16);
    softmax_kernel<<<blocks, 128, (size_t)((d->len + 15) & ~15), (cudaStream_t)stream>>>(*d, dl_rescale(d->out_exponent));
    count_launch();
    return check_launch("softmax");
}
