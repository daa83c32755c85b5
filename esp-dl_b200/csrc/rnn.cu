// GRU and LSTM over a whole sequence, batch 1, forward or bidirectional: the quantized branches of
// dl::module::GRU::forward_template (esp-dl/dl/module/include/dl_module_gru.hpp:114-256) and dl::module::LSTM::forward_template
// (esp-dl/dl/module/include/dl_module_lstm.hpp:125-300).  A recurrence has no parallelism across time steps, so the whole
// sequence is ONE launch of ONE thread block: per step the warps share the rows of the two matrix-vector products
// (base::mat_vec_dotprod, esp-dl/dl/base/dl_base_dotprod.hpp:36-43 with dotprod_c of dl_base_dotprod.cpp:8-42: an exact
// integer sum, then round(sum * 2^-shift) in fp32, saturated to int16), then the threads share the gate and state updates;
// the hidden and cell state, both int16 pre-activation vectors and the gate values live in shared memory between steps.
// Integer sums do not depend on the order of the additions; every fp32 operation of the gate arithmetic is issued as a
// separately rounded multiply or add in the reference's order.  The sigmoid / tanh tables (math::SigmoidLUT, math::TanhLUT,
// esp-dl/dl/math/include/dl_math.hpp:324-429) are built by the host with its own expf and only looked up here.
#include "common.cuh"

#include <mutex>

namespace espdl {

namespace {

struct RnnTables {
    const float *sig, *tanh;
    int sig_max, tanh_max;
};

__device__ __forceinline__ float sigmoid_lut(const RnnTables &t, int index)
{
    if (index >= 0)
        return index < t.sig_max ? t.sig[index] : t.sig[t.sig_max];
    return __fsub_rn(1.f, index > -t.sig_max ? t.sig[-index] : t.sig[t.sig_max]);
}

__device__ __forceinline__ float tanh_lut(const RnnTables &t, int index)
{
    if (index >= 0)
        return index < t.tanh_max ? t.tanh[index] : t.tanh[t.tanh_max];
    return -(index > -t.tanh_max ? t.tanh[-index] : t.tanh[t.tanh_max]);
}

// result[row] = sat16(round(dot(matrix[row], vector) * scale)) for the rows this warp owns
template <typename TM>
__device__ __forceinline__ void mat_vec(const TM *matrix, const int *vector_s, int16_t *result_s, int rows, int cols, float scale, int half_even,
                                        int warp, int lane, int nwarps)
{
    for (int r = warp; r < rows; r += nwarps) {
        const TM *row = matrix + (long long)r * cols;
        long long acc = 0;
        for (int c = lane; c < cols; c += 32) acc += (long long)((int)row[c] * vector_s[c]);
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) {
            // int8 products are summed in an int32, int16 products in an int64; both convert to fp32 before the scale
            const float f = sizeof(TM) == 1 ? __int2float_rn((int)acc) : __ll2float_rn(acc);
            result_s[r] = (int16_t)sat16(fround(__fmul_rn(f, scale), half_even));
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(512) rnn_kernel(espdl_rnn_desc d)
{
    extern __shared__ __align__(16) unsigned char smem[];
    const int H = d.hidden_size, G = d.op == ESPDL_RNN_GRU ? 3 : 4, GH = G * H;
    int *h_prev = (int *)smem;                 // H
    int *x_s = h_prev + H;                     // input_size
    float *gates = (float *)(x_s + d.input_size); // G * H
    int16_t *in_cache = (int16_t *)(gates + GH);  // G * H
    int16_t *hid_cache = in_cache + GH;           // G * H
    int16_t *c_prev = hid_cache + GH;             // H (LSTM)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
    const RnnTables tab = {d.sigmoid_table, d.tanh_table, d.sigmoid_max, d.tanh_max};
    const int he = d.round_mode == ESPDL_ROUND_HALF_EVEN;
    const float w_scale = dl_rescale(d.gate_exponent - (d.x_exponent + d.w_exponent));
    const float r_scale = dl_rescale(d.gate_exponent - (d.h_exponent + d.r_exponent));
    const float rescale_y = dl_rescale(d.y_exponent), rescale_c = dl_rescale(d.c_exponent);
    const T *x = (const T *)d.x;
    T *y = (T *)d.y, *y_h = (T *)d.y_h;
    const int lo = sizeof(T) == 1 ? -128 : -32768, hi = sizeof(T) == 1 ? 127 : 32767;

    for (int di = 0; di < d.directions; di++) {
        const T *w = (const T *)d.w + (long long)di * GH * d.input_size;
        const T *r = (const T *)d.r + (long long)di * GH * H;
        const int16_t *wb = d.b ? d.b + (long long)di * 2 * GH : nullptr, *rb = wb ? wb + GH : nullptr;
        for (int i = tid; i < H; i += blockDim.x) {
            h_prev[i] = d.initial_h ? (int)((const T *)d.initial_h)[di * H + i] : 0;
            c_prev[i] = d.initial_c ? d.initial_c[di * H + i] : (int16_t)0;
        }
        for (int step = 0; step < d.seq_length; step++) {
            const int t = di == 0 ? step : d.seq_length - 1 - step;
            for (int i = tid; i < d.input_size; i += blockDim.x) x_s[i] = (int)x[(long long)t * d.input_size + i];
            __syncthreads();
            mat_vec<T>(w, x_s, in_cache, GH, d.input_size, w_scale, he, warp, lane, nwarps);
            mat_vec<T>(r, h_prev, hid_cache, GH, H, r_scale, he, warp, lane, nwarps);
            __syncthreads();
            if (d.op == ESPDL_RNN_GRU) {
                // biases wrap in int16, as the reference's int16_t += does
                if (wb)
                    for (int i = tid; i < GH; i += blockDim.x) {
                        in_cache[i] = (int16_t)(in_cache[i] + wb[i]);
                        hid_cache[i] = (int16_t)(hid_cache[i] + rb[i]);
                    }
                __syncthreads();
                for (int i = tid; i < 2 * H; i += blockDim.x) gates[i] = sigmoid_lut(tab, (int)in_cache[i] + (int)hid_cache[i]); // z, r
                __syncthreads();
                for (int i = tid; i < H; i += blockDim.x) {
                    const float rg = gates[H + i];
                    const int index = fround(__fadd_rn((float)in_cache[2 * H + i], __fmul_rn(rg, (float)hid_cache[2 * H + i])), he);
                    const float n = tanh_lut(tab, index), z = gates[i];
                    float temp = __fmul_rn(__fmul_rn(__fsub_rn(1.f, z), n), rescale_y);
                    temp = __fadd_rn(temp, __fmul_rn(z, (float)h_prev[i]));
                    const int q = max(lo, min(hi, fround(temp, he)));
                    h_prev[i] = q;
                    y[((long long)t * d.directions + di) * H + i] = (T)q;
                }
            } else {
                for (int i = tid; i < GH; i += blockDim.x)
                    in_cache[i] = (int16_t)(in_cache[i] + (wb ? (int)wb[i] + (int)hid_cache[i] + (int)rb[i] : (int)hid_cache[i]));
                __syncthreads();
                for (int i = tid; i < H; i += blockDim.x) {
                    // gate order in W / R / B: input, output, forget, cell
                    const float ig = sigmoid_lut(tab, in_cache[i]), og = sigmoid_lut(tab, in_cache[H + i]);
                    const float fg = sigmoid_lut(tab, in_cache[2 * H + i]), gg = tanh_lut(tab, in_cache[3 * H + i]);
                    float temp = __fadd_rn(__fmul_rn(fg, (float)c_prev[i]), __fmul_rn(__fmul_rn(ig, gg), rescale_c));
                    const int16_t c = (int16_t)fround(temp, he); // the cell state is stored without saturation
                    c_prev[i] = c;
                    temp = __fmul_rn(__fmul_rn(og, tanh_lut(tab, c)), rescale_y);
                    const int q = max(lo, min(hi, fround(temp, he)));
                    h_prev[i] = q;
                    y[((long long)t * d.directions + di) * H + i] = (T)q;
                }
            }
            __syncthreads();
        }
        for (int i = tid; i < H; i += blockDim.x) {
            y_h[di * H + i] = (T)h_prev[i];
            if (d.op == ESPDL_RNN_LSTM && d.y_c)
                d.y_c[di * H + i] = c_prev[i];
        }
        __syncthreads();
    }
}

} // namespace

} // namespace espdl

using namespace espdl;

extern "C" int espdl_b200_rnn(const espdl_rnn_desc *d, void *stream)
{
    if (!d || !d->x || !d->w || !d->r || !d->y || !d->y_h || !d->sigmoid_table || !d->tanh_table || d->sigmoid_max < 1 || d->tanh_max < 1)
        return ESPDL_ERR_INVALID_ARG;
    if ((d->op != ESPDL_RNN_GRU && d->op != ESPDL_RNN_LSTM) || d->seq_length < 0 || d->input_size < 1 || d->hidden_size < 1 ||
        (d->directions != 1 && d->directions != 2))
        return ESPDL_ERR_INVALID_ARG;
    if (d->dtype != ESPDL_DTYPE_INT8 && d->dtype != ESPDL_DTYPE_INT16)
        return ESPDL_ERR_UNSUPPORTED;
    for (int e : {d->x_exponent, d->w_exponent, d->r_exponent, d->h_exponent, d->y_exponent, d->c_exponent, d->gate_exponent})
        if (e > 30 || e < -30)
            return ESPDL_ERR_INVALID_ARG;
    const int s1 = d->gate_exponent - (d->x_exponent + d->w_exponent), s2 = d->gate_exponent - (d->h_exponent + d->r_exponent);
    if (s1 > 30 || s1 < -30 || s2 > 30 || s2 < -30)
        return ESPDL_ERR_INVALID_ARG;
    const int G = d->op == ESPDL_RNN_GRU ? 3 : 4;
    const size_t smem = (size_t)(d->hidden_size + d->input_size) * 4 + (size_t)G * d->hidden_size * (4 + 2 + 2) + (size_t)d->hidden_size * 2 + 16;
    if (smem > 200 * 1024)
        return ESPDL_ERR_TOO_LARGE;
    static std::once_flag attr_once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(attr_once, [] {
        attr_err = cudaFuncSetAttribute(rnn_kernel<int8_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (attr_err == cudaSuccess)
            attr_err = cudaFuncSetAttribute(rnn_kernel<int16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    });
    if (attr_err != cudaSuccess)
        return set_cuda_error(attr_err, "cudaFuncSetAttribute(rnn_kernel)");
    if (d->dtype == ESPDL_DTYPE_INT8)
        rnn_kernel<int8_t><<<1, 512, smem, (cudaStream_t)stream>>>(*d);
    else
        rnn_kernel<int16_t><<<1, 512, smem, (cudaStream_t)stream>>>(*d);
    count_launch();
    return check_launch("rnn");
}
