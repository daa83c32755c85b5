// CUDA-core Conv2D for every shape the tensor-core tile kernel does not take
// (filters larger than 1x1, channel counts that are not a multiple of 16, strides,
// dilation, int16 with a large K).  One thread owns one output pixel and a group of
// OCT consecutive output channels, so each input value it loads feeds OCT MACs; the
// int8 path reads four input channels per 32-bit load and uses dp4a.
//
// Replaces dl::base::conv2d<> for those shapes
// (esp-dl/dl/base/dl_base_conv2d.cpp:141-162 MAC loop, esp-dl/dl/base/dl_base.hpp:951-1022
// border handling, esp-dl/dl/base/dl_base_activate_buffer.hpp:27-73 epilogue).
#include "common.cuh"

namespace espdl {

struct ConvParams {
    const void *in, *w, *bias;
    void *out;
    const int32_t *ew;
    const int8_t *lut;
    int lut_stride; // 0: one table, else entries between the tables of consecutive channels
    const int8_t *res; // optional residual added to the result (a folded Add), or null
    int rps;           // residual pixel stride
    int n, ih, iw, ic, oh, ow, oc, kh, kw, sh, sw, dh, dw, pt, pl, ips, ops;
    int e_shift_base; // out_exponent - in_exponent; shift = base - e_w
    int ew_scalar, per_channel, relu, half_even;
    long long total; // number of (pixel, oc-group) work items
    int groups;      // oc groups per pixel
};

template <int OCT, bool DP4A>
__global__ void __launch_bounds__(256) conv_s8_kernel(ConvParams p)
{
    const int8_t *__restrict__ in = (const int8_t *)p.in;
    const int8_t *__restrict__ w = (const int8_t *)p.w;
    const int32_t *__restrict__ bias = (const int32_t *)p.bias;
    int8_t *__restrict__ out = (int8_t *)p.out;
    const long long wstride = (long long)p.kh * p.kw * p.ic; // elements per output channel
    for (long long item = blockIdx.x * (long long)blockDim.x + threadIdx.x; item < p.total;
         item += (long long)gridDim.x * blockDim.x) {
        const int g = (int)(item % p.groups);
        const long long pix = item / p.groups;
        const int ox = (int)(pix % p.ow);
        const int oy = (int)((pix / p.ow) % p.oh);
        const int n = (int)(pix / ((long long)p.ow * p.oh));
        const int oc0 = g * OCT;
        int32_t acc[OCT];
#pragma unroll
        for (int j = 0; j < OCT; j++) acc[j] = 0;
        for (int ky = 0; ky < p.kh; ky++) {
            const int iy = oy * p.sh + ky * p.dh - p.pt;
            if (iy < 0 || iy >= p.ih)
                continue;
            for (int kx = 0; kx < p.kw; kx++) {
                const int ix = ox * p.sw + kx * p.dw - p.pl;
                if (ix < 0 || ix >= p.iw)
                    continue;
                const int8_t *ip = in + (((long long)n * p.ih + iy) * p.iw + ix) * p.ips;
                const int8_t *wp = w + (long long)oc0 * wstride + ((long long)ky * p.kw + kx) * p.ic;
                if (DP4A) {
                    const int *ip4 = (const int *)ip;
                    for (int c = 0; c < p.ic / 4; c++) {
                        const int a = __ldg(ip4 + c);
#pragma unroll
                        for (int j = 0; j < OCT; j++) {
                            if (oc0 + j < p.oc)
                                acc[j] = __dp4a(a, __ldg((const int *)(wp + j * wstride) + c), acc[j]);
                        }
                    }
                } else {
                    for (int c = 0; c < p.ic; c++) {
                        const int a = ip[c];
#pragma unroll
                        for (int j = 0; j < OCT; j++) {
                            if (oc0 + j < p.oc)
                                acc[j] += a * (int)wp[j * wstride + c];
                        }
                    }
                }
            }
        }
        int8_t *op = out + pix * p.ops + oc0;
#pragma unroll
        for (int j = 0; j < OCT; j++) {
            const int oc = oc0 + j;
            if (oc < p.oc) {
                const int e = p.per_channel ? p.ew[oc] : p.ew_scalar;
                const int shift = max(-31, min(31, p.e_shift_base - e));
                int32_t q = requant8(acc[j], bias ? bias[oc] : 0, shift, p.relu, p.half_even);
                if (p.lut)
                    q = p.lut[(long long)oc * p.lut_stride + ((uint8_t)q ^ 0x80u)];
                if (p.res)
                    q = sat8(q + (int)p.res[pix * p.rps + oc]);
                op[j] = (int8_t)q;
            }
        }
    }
}

template <int OCT>
__global__ void __launch_bounds__(256) conv_s16_kernel(ConvParams p)
{
    const int16_t *__restrict__ in = (const int16_t *)p.in;
    const int16_t *__restrict__ w = (const int16_t *)p.w;
    const long long *__restrict__ bias = (const long long *)p.bias;
    int16_t *__restrict__ out = (int16_t *)p.out;
    const long long wstride = (long long)p.kh * p.kw * p.ic;
    for (long long item = blockIdx.x * (long long)blockDim.x + threadIdx.x; item < p.total;
         item += (long long)gridDim.x * blockDim.x) {
        const int g = (int)(item % p.groups);
        const long long pix = item / p.groups;
        const int ox = (int)(pix % p.ow);
        const int oy = (int)((pix / p.ow) % p.oh);
        const int n = (int)(pix / ((long long)p.ow * p.oh));
        const int oc0 = g * OCT;
        long long acc[OCT];
#pragma unroll
        for (int j = 0; j < OCT; j++) acc[j] = 0;
        for (int ky = 0; ky < p.kh; ky++) {
            const int iy = oy * p.sh + ky * p.dh - p.pt;
            if (iy < 0 || iy >= p.ih)
                continue;
            for (int kx = 0; kx < p.kw; kx++) {
                const int ix = ox * p.sw + kx * p.dw - p.pl;
                if (ix < 0 || ix >= p.iw)
                    continue;
                const int16_t *ip = in + (((long long)n * p.ih + iy) * p.iw + ix) * p.ips;
                const int16_t *wp = w + (long long)oc0 * wstride + ((long long)ky * p.kw + kx) * p.ic;
                for (int c = 0; c < p.ic; c++) {
                    const int a = ip[c];
#pragma unroll
                    for (int j = 0; j < OCT; j++) {
                        if (oc0 + j < p.oc)
                            acc[j] += (long long)(a * (int)wp[j * wstride + c]); // |a*w| < 2^31: exact in int32
                    }
                }
            }
        }
        int16_t *op = out + pix * p.ops + oc0;
#pragma unroll
        for (int j = 0; j < OCT; j++) {
            const int oc = oc0 + j;
            if (oc < p.oc) {
                const int e = p.per_channel ? p.ew[oc] : p.ew_scalar;
                const int shift = max(-62, min(62, p.e_shift_base - e));
                op[j] = (int16_t)requant16(acc[j], bias ? bias[oc] : 0ll, shift, p.relu, p.half_even);
            }
        }
    }
}

// Stem-style convolutions (a handful of input channels, e.g. the 3-channel 3x3 stride-2 first layer of an image
// network): K = kh*kw*in_c is tiny, so the whole filter bank sits in shared memory packed four taps per 32-bit
// word, each thread gathers the K input bytes of ONE output pixel into registers once and then produces every
// output channel of that pixel with dp4a.  Output bytes of a pixel are contiguous, so stores are 128-bit.
constexpr int SMALL_MAX_WORDS = 16; // K <= 64
constexpr int SMALL_MAX_OC = 64;

template <int KH, int KW, int IC>
__global__ void __launch_bounds__(256) conv_s8_small_k_kernel(ConvParams p)
{
    __shared__ int w_s[SMALL_MAX_OC * SMALL_MAX_WORDS];
    __shared__ int bias_s[SMALL_MAX_OC];
    __shared__ int shift_s[SMALL_MAX_OC];
    constexpr int K = KH * KW * IC;
    constexpr int words = (K + 3) / 4;
    static_assert(words <= SMALL_MAX_WORDS, "filter too large for the small-K kernel");
    const int8_t *__restrict__ in = (const int8_t *)p.in;
    const int8_t *__restrict__ w = (const int8_t *)p.w;
    for (int i = threadIdx.x; i < p.oc * words; i += blockDim.x) {
        const int oc = i / words, wd = i % words;
        uint32_t v = 0;
        for (int b = 0; b < 4; b++) {
            const int k = wd * 4 + b;
            if (k < K)
                v |= ((uint32_t)(uint8_t)w[(long long)oc * K + k]) << (8 * b);
        }
        w_s[i] = (int)v;
    }
    for (int oc = threadIdx.x; oc < p.oc; oc += blockDim.x) {
        bias_s[oc] = p.bias ? ((const int32_t *)p.bias)[oc] : 0;
        const int e = p.per_channel ? p.ew[oc] : p.ew_scalar;
        shift_s[oc] = max(-31, min(31, p.e_shift_base - e));
    }
    __syncthreads();
    const long long pixels = (long long)p.n * p.oh * p.ow;
    const bool vec_store = (p.oc % 16 == 0) && (p.ops % 16 == 0) && (((uintptr_t)p.out) % 16 == 0);
    for (long long pix = blockIdx.x * (long long)blockDim.x + threadIdx.x; pix < pixels; pix += (long long)gridDim.x * blockDim.x) {
        const int ox = (int)(pix % p.ow);
        const int oy = (int)((pix / p.ow) % p.oh);
        const int n = (int)(pix / ((long long)p.ow * p.oh));
        int a[words];
#pragma unroll
        for (int i = 0; i < words; i++) a[i] = 0;
        // gather the K input bytes in filter order (ky, kx, c); taps outside the image stay 0
#pragma unroll
        for (int ky = 0; ky < KH; ky++) {
            const int iy = oy * p.sh + ky * p.dh - p.pt;
#pragma unroll
            for (int kx = 0; kx < KW; kx++) {
                const int ix = ox * p.sw + kx * p.dw - p.pl;
                const bool inside = iy >= 0 && iy < p.ih && ix >= 0 && ix < p.iw;
                const int8_t *ip = in + (((long long)n * p.ih + iy) * p.iw + ix) * p.ips;
#pragma unroll
                for (int c = 0; c < IC; c++) {
                    constexpr int dummy = 0;
                    (void)dummy;
                    const int k = (ky * KW + kx) * IC + c; // compile-time after unrolling: a[] stays in registers
                    const uint32_t v = inside ? (uint32_t)(uint8_t)__ldg(ip + c) : 0u;
                    a[k >> 2] |= (int)(v << (8 * (k & 3)));
                }
            }
        }
        int8_t *op = (int8_t *)p.out + pix * p.ops;
        for (int oc0 = 0; oc0 < p.oc; oc0 += 16) {
            uint32_t pk[4] = {0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const int oc = oc0 + j;
                if (oc < p.oc) {
                    int acc = 0;
                    const int *wr = w_s + oc * words;
#pragma unroll
                    for (int i = 0; i < words; i++) acc = __dp4a(a[i], wr[i], acc);
                    int q = requant8(acc, bias_s[oc], shift_s[oc], p.relu, p.half_even);
                    if (p.lut)
                        q = p.lut[(long long)oc * p.lut_stride + ((uint8_t)q ^ 0x80u)];
                    pk[j >> 2] |= ((uint32_t)q & 0xffu) << (8 * (j & 3));
                }
            }
            if (vec_store) {
                *(uint4 *)(op + oc0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            } else {
                for (int j = 0; j < 16 && oc0 + j < p.oc; j++) op[oc0 + j] = (int8_t)(pk[j >> 2] >> (8 * (j & 3)));
            }
        }
    }
}

int conv2d_simt(const espdl_conv_desc &d, cudaStream_t s)
{
    ConvParams p;
    p.res = (const int8_t *)d.residual, p.rps = d.residual_pixel_stride ? d.residual_pixel_stride : d.out_c;
    p.in = d.input, p.w = d.filter, p.bias = d.bias, p.out = d.output, p.ew = d.filter_exponents, p.lut = d.lut, p.lut_stride = d.lut_channel_stride;
    p.n = d.n, p.ih = d.in_h, p.iw = d.in_w, p.ic = d.in_c, p.oh = d.out_h, p.ow = d.out_w, p.oc = d.out_c;
    p.kh = d.kh, p.kw = d.kw, p.sh = d.stride_h, p.sw = d.stride_w, p.dh = d.dilation_h, p.dw = d.dilation_w;
    p.pt = d.pad_top, p.pl = d.pad_left;
    p.ips = d.in_pixel_stride ? d.in_pixel_stride : d.in_c;
    p.ops = d.out_pixel_stride ? d.out_pixel_stride : d.out_c;
    p.e_shift_base = d.out_exponent - d.in_exponent;
    p.ew_scalar = d.filter_exponent, p.per_channel = d.per_channel;
    p.relu = d.activation == ESPDL_ACT_RELU, p.half_even = d.round_mode == ESPDL_ROUND_HALF_EVEN;
    constexpr int OCT = 4;
    p.groups = (d.out_c + OCT - 1) / OCT;
    p.total = (long long)d.n * d.out_h * d.out_w * p.groups;
    const int threads = 256;
    long long blocks = (p.total + threads - 1) / threads;
    const long long max_blocks = (long long)num_sms() * 32;
    if (blocks > max_blocks)
        blocks = max_blocks;
    if (d.dtype == ESPDL_DTYPE_INT8 && d.out_c <= SMALL_MAX_OC && d.kh == 3 && d.kw == 3 && (d.in_c == 3 || d.in_c == 1 || d.in_c == 4)) {
        const long long pixels = (long long)d.n * d.out_h * d.out_w;
        const unsigned grid = (unsigned)min((pixels + threads - 1) / threads, max_blocks);
        if (d.in_c == 3)
            conv_s8_small_k_kernel<3, 3, 3><<<grid, threads, 0, s>>>(p);
        else if (d.in_c == 1)
            conv_s8_small_k_kernel<3, 3, 1><<<grid, threads, 0, s>>>(p);
        else
            conv_s8_small_k_kernel<3, 3, 4><<<grid, threads, 0, s>>>(p);
    } else if (d.dtype == ESPDL_DTYPE_INT8) {
        const bool dp4a = d.in_c % 4 == 0 && p.ips % 4 == 0 && ((uintptr_t)d.input % 4) == 0 && ((uintptr_t)d.filter % 4) == 0;
        if (dp4a)
            conv_s8_kernel<OCT, true><<<(unsigned)blocks, threads, 0, s>>>(p);
        else
            conv_s8_kernel<OCT, false><<<(unsigned)blocks, threads, 0, s>>>(p);
    } else {
        conv_s16_kernel<OCT><<<(unsigned)blocks, threads, 0, s>>>(p);
    }
    count_launch();
    return check_launch("conv2d_simt");
}

} // namespace espdl
