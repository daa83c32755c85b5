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
    const int he = d.round_mode == ESPDL_ROUND_HALF_EVEN;
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
                ((int8_t *)d.output)[oi] = (int8_t)sat8(fround(__fmul_rn(y, out_rescale), he));
            else
                ((int16_t *)d.output)[oi] = (int16_t)sat16(fround(__fmul_rn(y, out_rescale), he));
        }
    }
}

// The same arithmetic with the rows side by side: a block stages R rows in shared memory (row pitch an odd number of
// words, so that thread r reading byte i of row r meets no bank conflict), thread r adds row r's exponentials in index
// order - R ordered sums run at once instead of one -, then all threads write the R x len results.  Used whenever at
// least 32 rows fit into shared memory; the kernel above keeps the long rows.
__global__ void __launch_bounds__(256) softmax_rows_kernel(espdl_softmax_desc d, float out_rescale, int R, int pitch)
{
    __shared__ float table[256];
    extern __shared__ __align__(16) unsigned char sm[];
    float *sums = (float *)sm;               // R
    int8_t *rows = (int8_t *)(sums + R);     // R x pitch
    for (int i = threadIdx.x; i < 256; i += blockDim.x) table[i] = d.exp_table[i];
    const int inner = d.inner > 1 ? d.inner : 1;
    const float in_scale = dl_scale(d.in_exponent);
    const int he = d.round_mode == ESPDL_ROUND_HALF_EVEN;
    const int groups = (d.rows + R - 1) / R;
    for (int g = blockIdx.x; g < groups; g += gridDim.x) {
        const int r0 = g * R, nr = min(R, d.rows - r0);
        __syncthreads();
        const bool words = inner == 1 && d.len % 4 == 0 && (((uintptr_t)d.input) & 3) == 0; // whole 32-bit words per row
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5, len4 = d.len >> 2;
        if (words) {
            // a warp per row, a word per lane: no index divisions, 128-byte global reads
            for (int rr = warp; rr < nr; rr += nwarps) {
                const uint32_t *src = (const uint32_t *)(d.input + (long long)(r0 + rr) * d.len);
                uint32_t *dst = (uint32_t *)(rows + rr * pitch);
                for (int i = lane; i < len4; i += 32) dst[i] = src[i];
            }
        } else if (inner == 1) {
            // rows r0 .. r0 + nr - 1 are one contiguous span of nr * len bytes
            const int8_t *src = d.input + (long long)r0 * d.len;
            for (int e = threadIdx.x; e < nr * d.len; e += blockDim.x) rows[(e / d.len) * pitch + e % d.len] = src[e];
        } else {
            for (int e = threadIdx.x; e < nr * d.len; e += blockDim.x) {
                const int rr = e % nr, i = e / nr, r = r0 + rr; // neighbouring threads: neighbouring rows = neighbouring bytes
                rows[rr * pitch + i] = d.input[(long long)(r / inner) * d.len * inner + (r % inner) + (long long)i * inner];
            }
        }
        __syncthreads();
        if ((int)threadIdx.x < nr) {
            const int8_t *row = rows + threadIdx.x * pitch;
            float sum = 0.f;
            for (int i = 0; i < d.len; i++) sum = __fadd_rn(sum, table[row[i] + 128]);
            sums[threadIdx.x] = d.log ? logf(sum) : sum;
        }
        __syncthreads();
        if (words && d.out_dtype != ESPDL_DTYPE_INT16) {
            for (int rr = warp; rr < nr; rr += nwarps) {
                const uint32_t *src = (const uint32_t *)(rows + rr * pitch);
                const float sum = sums[rr];
                const long long o0 = (long long)(r0 + rr) * d.len;
                for (int i = lane; i < len4; i += 32) {
                    const uint32_t w = src[i];
                    float y[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const int x = (int)(int8_t)(w >> (8 * j));
                        y[j] = d.log ? __fsub_rn(__fmul_rn(in_scale, (float)x), sum) : __fdiv_rn(table[x + 128], sum);
                    }
                    if (d.out_dtype == ESPDL_DTYPE_FLOAT) {
                        float *op = (float *)d.output + o0 + 4 * i;
                        if ((((uintptr_t)op) & 15) == 0)
                            *(float4 *)op = make_float4(y[0], y[1], y[2], y[3]);
                        else
                            op[0] = y[0], op[1] = y[1], op[2] = y[2], op[3] = y[3];
                    } else {
                        uint32_t q = 0;
#pragma unroll
                        for (int j = 0; j < 4; j++) q |= ((uint32_t)sat8(fround(__fmul_rn(y[j], out_rescale), he)) & 0xffu) << (8 * j);
                        int8_t *op = (int8_t *)d.output + o0 + 4 * i;
                        if ((((uintptr_t)op) & 3) == 0)
                            *(uint32_t *)op = q;
                        else
                            op[0] = (int8_t)q, op[1] = (int8_t)(q >> 8), op[2] = (int8_t)(q >> 16), op[3] = (int8_t)(q >> 24);
                    }
                }
            }
            continue;
        }
        for (int e = threadIdx.x; e < nr * d.len; e += blockDim.x) {
            int rr, i;
            if (inner == 1)
                rr = e / d.len, i = e % d.len;
            else
                rr = e % nr, i = e / nr;
            const int r = r0 + rr;
            const int x = rows[rr * pitch + i];
            const float sum = sums[rr];
            const float y = d.log ? __fsub_rn(__fmul_rn(in_scale, (float)x), sum) : __fdiv_rn(table[x + 128], sum);
            const long long oi = (long long)(r / inner) * d.len * inner + (r % inner) + (long long)i * inner;
            if (d.out_dtype == ESPDL_DTYPE_FLOAT)
                ((float *)d.output)[oi] = y;
            else if (d.out_dtype == ESPDL_DTYPE_INT8)
                ((int8_t *)d.output)[oi] = (int8_t)sat8(fround(__fmul_rn(y, out_rescale), he));
            else
                ((int16_t *)d.output)[oi] = (int16_t)sat16(fround(__fmul_rn(y, out_rescale), he));
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
    // rows side by side when at least 32 of them fit into 40 KB of shared memory
    const int pitch = (((d->len + 3) / 4) | 1) * 4;
    const int fit = (40 * 1024) / (pitch + 4);
    if (fit >= 32 && d->rows >= 64) {
        const int R = min(256, fit);
        const int groups = (d->rows + R - 1) / R;
        softmax_rows_kernel<<<min(groups, num_sms() * 8), 256, (size_t)R * (pitch + 4) + 16, (cudaStream_t)stream>>>(*d, dl_rescale(d->out_exponent), R, pitch);
        count_launch();
        return check_launch("softmax_rows");
    }
    const int blocks = min(d->rows, num_sms() * 16);
    softmax_kernel<<<blocks, 128, (size_t)((d->len + 15) & ~15), (cudaStream_t)stream>>>(*d, dl_rescale(d->out_exponent));
    count_launch();
    return check_launch("softmax");
}
