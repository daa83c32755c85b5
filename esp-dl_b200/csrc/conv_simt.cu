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
                    q = p.lut[(uint8_t)q ^ 0x80u];
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

int conv2d_simt(const espdl_conv_desc &d, cudaStream_t s)
{
    ConvParams p;
    p.in = d.input, p.w = d.filter, p.bias = d.bias, p.out = d.output, p.ew = d.filter_exponents, p.lut = d.lut;
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
    if (d.dtype == ESPDL_DTYPE_INT8) {
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
