// RMSNormalization and LayerNormalization over the trailing axes of an int8 / int16 tensor.
// Replaces dl::module::RMSNormalization::forward_int8 / forward_int16 with dl::base::rms_norm
// (esp-dl/dl/module/include/dl_module_rms_normalization.hpp:57-113, esp-dl/dl/base/dl_base_norm.cpp:9-38) and the
// quantized branch of dl::module::LayerNormalization::forward_template
// (esp-dl/dl/module/include/dl_module_layer_normalization.hpp:141-214).
//
// A warp owns one row.  Integer sums (the row sum, the sum of squares) are exact, so the lanes split them and combine
// with shuffles.  LayerNormalization's variance is an fp32 sum whose result depends on the order of the additions: the
// lanes compute the squared differences of 32 consecutive elements in parallel and then every lane adds the 32 values
// in element order, so the sum is the reference's sequential sum bit for bit.  Every fp32 product, sum and quotient is
// rounded on its own (no fused multiply-add), as in the reference built without contraction.
#include "common.cuh"

namespace espdl {

namespace {

struct NormParams {
    const void *in, *scale, *bias;
    void *out, *mean, *inv_std;
    int op, half_even, len;
    long long rows;
    float in_scale, out_rescale, scale_scale, bias_scale, mean_rescale, inv_std_rescale, epsilon;
};

// math::sqrt_newton (esp-dl/dl/math/include/dl_math.hpp:83-97); the iteration ends by itself, the cap only bounds it
__device__ __forceinline__ float sqrt_newton_dev(float x)
{
    if (x == 0.f)
        return 0.f;
    float r = x;
    for (int it = 0; it < 100; it++) {
        const float last = r;
        r = __fmul_rn(__fadd_rn(last, __fdiv_rn(x, last)), 0.5f);
        if (!(fabsf(__fsub_rn(r, last)) > 0.00001f))
            break;
    }
    return r;
}

template <typename T>
__device__ __forceinline__ void store_q(T *p, long long i, int q)
{
    p[i] = (T)(sizeof(T) == 1 ? sat8(q) : sat16(q));
}

// V consecutive elements of a row as one 32-bit word: 4 int8 or 2 int16.
template <typename T>
struct Word {
    static constexpr int V = 4 / (int)sizeof(T);
    uint32_t w;
    __device__ __forceinline__ int get(int i) const
    {
        return sizeof(T) == 1 ? (int)(int8_t)(w >> (8 * i)) : (int)(int16_t)(w >> (16 * i));
    }
    __device__ __forceinline__ void set(int i, int q)
    {
        if (sizeof(T) == 1)
            w |= ((uint32_t)sat8(q) & 0xffu) << (8 * i);
        else
            w |= ((uint32_t)sat16(q) & 0xffffu) << (16 * i);
    }
};

// Rows whose length is a multiple of V and whose pointers are word aligned: every lane moves whole words.  The
// variance terms of 32 * V consecutive elements go through shared memory (one float4 / float2 per lane) and every lane
// then adds them in element order from broadcast reads, which costs a quarter of the shuffles of the scalar form.
template <typename T>
__device__ __forceinline__ void norm_row_words(const NormParams &p, const T *x, T *y, long long row, int lane, float *stage)
{
    constexpr int V = Word<T>::V;
    const int words = p.len / V;
    const uint32_t *xw = (const uint32_t *)x;
    uint32_t *yw = (uint32_t *)y;
    if (p.op == ESPDL_NORM_RMS) {
        long long ss = 0;
        for (int j = lane; j < words; j += 32) {
            Word<T> a{xw[j]};
#pragma unroll
            for (int i = 0; i < V; i++) ss += (long long)(a.get(i) * a.get(i));
        }
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float fsum = sizeof(T) == 1 ? __int2float_rn((int)ss) : __ll2float_rn(ss);
        const float mean_sq = __fdiv_rn(__fmul_rn(fsum, __fmul_rn(p.in_scale, p.in_scale)), __int2float_rn(p.len));
        float rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_sq, p.epsilon)));
        rms = __fmul_rn(rms, __fmul_rn(p.in_scale, p.out_rescale));
        const float *sc = (const float *)p.scale;
        const bool sc_vec = ((uintptr_t)sc % (4 * V)) == 0;
        for (int j = lane; j < words; j += 32) {
            Word<T> a{xw[j]}, r{0u};
            float s4[V];
            if (sc_vec && V == 4) {
                const float4 t = *(const float4 *)(sc + j * V);
                s4[0] = t.x, s4[1] = t.y, s4[V - 2] = t.z, s4[V - 1] = t.w;
            } else if (sc_vec) {
                const float2 t = *(const float2 *)(sc + j * V);
                s4[0] = t.x, s4[1] = t.y;
            } else {
#pragma unroll
                for (int i = 0; i < V; i++) s4[i] = sc[j * V + i];
            }
#pragma unroll
            for (int i = 0; i < V; i++) r.set(i, fround(__fmul_rn(__fmul_rn(__int2float_rn(a.get(i)), rms), s4[i]), p.half_even));
            yw[j] = r.w;
        }
        return;
    }
    int sum = 0;
    for (int j = lane; j < words; j += 32) {
        Word<T> a{xw[j]};
#pragma unroll
        for (int i = 0; i < V; i++) sum += a.get(i);
    }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    float mean = (float)((double)sum * 1.0 / (double)p.len);
    if (p.mean && lane == 0)
        store_q((T *)p.mean, row, fround(__fmul_rn(__fmul_rn(mean, p.mean_rescale), p.in_scale), p.half_even));
    float var = 0.f;
    for (int base = 0; base < words; base += 32) {
        const int j = base + lane;
        float d2[V];
#pragma unroll
        for (int i = 0; i < V; i++) d2[i] = 0.f;
        if (j < words) {
            Word<T> a{xw[j]};
#pragma unroll
            for (int i = 0; i < V; i++) {
                const float d = __fsub_rn(__int2float_rn(a.get(i)), mean);
                d2[i] = __fmul_rn(d, d);
            }
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < V; i++) stage[lane * V + i] = d2[i];
        __syncwarp();
        const int n = min(32, words - base) * V;
        for (int k = 0; k < n; k += V) { // one broadcast read of V terms, added in element order
            if (V == 4) {
                const float4 t = *(const float4 *)(stage + k);
                var = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(var, t.x), t.y), t.z), t.w);
            } else {
                const float2 t = *(const float2 *)(stage + k);
                var = __fadd_rn(__fadd_rn(var, t.x), t.y);
            }
        }
    }
    mean = __fmul_rn(mean, p.in_scale);
    var = __fmul_rn(var, __fmul_rn(p.in_scale, p.in_scale));
    var = __fdiv_rn(var, __int2float_rn(p.len));
    const float inv_std = __fdiv_rn(1.0f, sqrt_newton_dev(__fadd_rn(var, p.epsilon)));
    if (p.inv_std && lane == 0)
        store_q((T *)p.inv_std, row, fround(__fmul_rn(inv_std, p.inv_std_rescale), p.half_even));
    const T *sc = (const T *)p.scale, *bi = (const T *)p.bias;
    for (int j = lane; j < words; j += 32) {
        Word<T> a{xw[j]}, r{0u};
#pragma unroll
        for (int i = 0; i < V; i++) {
            const int e = j * V + i;
            const float xv = __fmul_rn(__int2float_rn(a.get(i)), p.in_scale);
            const float normalized = __fmul_rn(__fsub_rn(xv, mean), inv_std);
            const float sv = sc ? __fmul_rn(__int2float_rn((int)sc[e]), p.scale_scale) : 1.0f;
            const float bv = bi ? __fmul_rn(__int2float_rn((int)bi[e]), p.bias_scale) : 0.0f;
            r.set(i, fround(__fmul_rn(__fadd_rn(__fmul_rn(normalized, sv), bv), p.out_rescale), p.half_even));
        }
        yw[j] = r.w;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) norm_kernel(NormParams p)
{
    __shared__ __align__(16) float stage_all[8][128];
    const bool words_ok = p.len % Word<T>::V == 0 && ((uintptr_t)p.in % 4) == 0 && ((uintptr_t)p.out % 4) == 0;
    const int lane = threadIdx.x & 31;
    const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5, warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long row = warp; row < p.rows; row += warps) {
        const T *x = (const T *)p.in + row * p.len;
        T *y = (T *)p.out + row * p.len;
        if (words_ok) {
            norm_row_words<T>(p, x, y, row, lane, stage_all[threadIdx.x >> 5]);
            continue;
        }
        if (p.op == ESPDL_NORM_RMS) {
            // int8: int32 sum of squares (as dl::base::reduce_l2 returns it), int16: int64
            long long ss = 0;
            for (int j = lane; j < p.len; j += 32) ss += (long long)((int)x[j] * (int)x[j]);
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float fsum = sizeof(T) == 1 ? __int2float_rn((int)ss) : __ll2float_rn(ss);
            const float mean_sq = __fdiv_rn(__fmul_rn(fsum, __fmul_rn(p.in_scale, p.in_scale)), __int2float_rn(p.len));
            float rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_sq, p.epsilon)));
            rms = __fmul_rn(rms, __fmul_rn(p.in_scale, p.out_rescale));
            const float *sc = (const float *)p.scale;
            for (int j = lane; j < p.len; j += 32)
                store_q(y, j, fround(__fmul_rn(__fmul_rn(__int2float_rn((int)x[j]), rms), sc[j]), p.half_even));
        } else {
            int sum = 0;
            for (int j = lane; j < p.len; j += 32) sum += (int)x[j];
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            float mean = (float)((double)sum * 1.0 / (double)p.len);
            if (p.mean && lane == 0)
                store_q((T *)p.mean, row, fround(__fmul_rn(__fmul_rn(mean, p.mean_rescale), p.in_scale), p.half_even));
            float var = 0.f;
            for (int base = 0; base < p.len; base += 32) {
                const int j = base + lane;
                float d2 = 0.f;
                if (j < p.len) {
                    const float d = __fsub_rn(__int2float_rn((int)x[j]), mean);
                    d2 = __fmul_rn(d, d);
                }
                const int n = min(32, p.len - base);
                for (int k = 0; k < n; k++) var = __fadd_rn(var, __shfl_sync(0xffffffffu, d2, k));
            }
            mean = __fmul_rn(mean, p.in_scale);
            var = __fmul_rn(var, __fmul_rn(p.in_scale, p.in_scale));
            var = __fdiv_rn(var, __int2float_rn(p.len));
            const float inv_std = __fdiv_rn(1.0f, sqrt_newton_dev(__fadd_rn(var, p.epsilon)));
            if (p.inv_std && lane == 0)
                store_q((T *)p.inv_std, row, fround(__fmul_rn(inv_std, p.inv_std_rescale), p.half_even));
            const T *sc = (const T *)p.scale, *bi = (const T *)p.bias;
            for (int j = lane; j < p.len; j += 32) {
                const float xv = __fmul_rn(__int2float_rn((int)x[j]), p.in_scale);
                const float normalized = __fmul_rn(__fsub_rn(xv, mean), inv_std);
                const float sv = sc ? __fmul_rn(__int2float_rn((int)sc[j]), p.scale_scale) : 1.0f;
                const float bv = bi ? __fmul_rn(__int2float_rn((int)bi[j]), p.bias_scale) : 0.0f;
                const float r = __fadd_rn(__fmul_rn(normalized, sv), bv);
                store_q(y, j, fround(__fmul_rn(r, p.out_rescale), p.half_even));
            }
        }
    }
}

} // namespace

} // namespace espdl

using namespace espdl;

extern "C" int espdl_b200_norm(const espdl_norm_desc *d, void *stream)
{
    if (!d || !d->input || !d->output || d->rows < 0 || d->len <= 0)
        return ESPDL_ERR_INVALID_ARG;
    if (d->op != ESPDL_NORM_RMS && d->op != ESPDL_NORM_LAYER && d->op != ESPDL_NORM_LP)
        return ESPDL_ERR_INVALID_ARG;
    if (d->op == ESPDL_NORM_RMS && !d->scale)
        return ESPDL_ERR_INVALID_ARG;
    if (d->dtype != ESPDL_DTYPE_INT8 && d->dtype != ESPDL_DTYPE_INT16)
        return ESPDL_ERR_UNSUPPORTED;
    for (int e : {d->in_exponent, d->out_exponent, d->scale_exponent, d->bias_exponent, d->mean_exponent, d->inv_std_dev_exponent})
        if (e > 30 || e < -30)
            return ESPDL_ERR_INVALID_ARG;
    if (d->rows == 0)
        return ESPDL_OK;
    if (d->op == ESPDL_NORM_LP)
        return lp_norm_op(*d, (cudaStream_t)stream);
    NormParams p;
    p.in = d->input, p.out = d->output, p.scale = d->scale, p.bias = d->bias, p.mean = d->mean, p.inv_std = d->inv_std_dev;
    p.op = d->op, p.half_even = d->round_mode == ESPDL_ROUND_HALF_EVEN, p.len = d->len, p.rows = d->rows;
    p.in_scale = dl_scale(d->in_exponent), p.out_rescale = dl_rescale(d->out_exponent);
    p.scale_scale = dl_scale(d->scale_exponent), p.bias_scale = dl_scale(d->bias_exponent);
    p.mean_rescale = dl_rescale(d->mean_exponent), p.inv_std_rescale = dl_rescale(d->inv_std_dev_exponent);
    p.epsilon = d->epsilon;
    const long long blocks = (d->rows + 7) / 8; // eight rows (warps) per block
    const unsigned grid = (unsigned)min(blocks, (long long)num_sms() * 8);
    if (d->dtype == ESPDL_DTYPE_INT8)
        norm_kernel<int8_t><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
    else
        norm_kernel<int16_t><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
    count_launch();
    return check_launch("norm");
}
