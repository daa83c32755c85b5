// DepthwiseConv2D (group == channels), int8 and int16.
// Replaces dl::base::depthwise_conv2d<> (esp-dl/dl/base/dl_base_depthwise_conv2d.cpp:47-66,
// shell esp-dl/dl/base/dl_base.hpp:1209-2107): out[y,x,c] = epilogue(sum_{ky,kx} in[..,c] * w[ky,kx,c] + bias[c]).
//
// The op is bandwidth bound (9 MACs per byte read): the int8 kernel moves 16 channels per
// thread with 128-bit loads and stores; consecutive threads own consecutive 16-channel
// chunks of one pixel, so a warp reads and writes contiguous 512-byte runs of the NHWC tensor.
// The filter taps, bias and per-channel shifts of a chunk are the same for every pixel and
// stay resident in L1.
#include "common.cuh"

namespace espdl {

struct DwParams {
    const void *in, *w, *bias;
    void *out;
    const int32_t *ew;
    const int8_t *lut;
    int n, ih, iw, c, oh, ow, kh, kw, sh, sw, dh, dw, pt, pl, ips, ops;
    int e_shift_base, ew_scalar, per_channel, relu, half_even;
    long long total;
    int chunks;
};

__device__ __forceinline__ int sbyte(uint32_t x, int i) { return (int)(int8_t)(x >> (8 * i)); }

__global__ void __launch_bounds__(256) dw_s8_vec16_kernel(DwParams p)
{
    const int8_t *__restrict__ in = (const int8_t *)p.in;
    const int8_t *__restrict__ w = (const int8_t *)p.w;
    const int32_t *__restrict__ bias = (const int32_t *)p.bias;
    int8_t *__restrict__ out = (int8_t *)p.out;
    for (long long item = blockIdx.x * (long long)blockDim.x + threadIdx.x; item < p.total;
         item += (long long)gridDim.x * blockDim.x) {
        const int ch = (int)(item % p.chunks) * 16;
        const long long pix = item / p.chunks;
        const int ox = (int)(pix % p.ow);
        const int oy = (int)((pix / p.ow) % p.oh);
        const int n = (int)(pix / ((long long)p.ow * p.oh));
        int32_t acc[16];
#pragma unroll
        for (int j = 0; j < 16; j++) acc[j] = 0;
        for (int ky = 0; ky < p.kh; ky++) {
            const int iy = oy * p.sh + ky * p.dh - p.pt;
            if (iy < 0 || iy >= p.ih)
                continue;
            for (int kx = 0; kx < p.kw; kx++) {
                const int ix = ox * p.sw + kx * p.dw - p.pl;
                if (ix < 0 || ix >= p.iw)
                    continue;
                const uint4 a = __ldg((const uint4 *)(in + (((long long)n * p.ih + iy) * p.iw + ix) * p.ips + ch));
                const uint4 b = __ldg((const uint4 *)(w + ((long long)ky * p.kw + kx) * p.c + ch));
                const uint32_t av[4] = {a.x, a.y, a.z, a.w};
                const uint32_t bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                for (int q = 0; q < 4; q++)
#pragma unroll
                    for (int i = 0; i < 4; i++) acc[q * 4 + i] += sbyte(av[q], i) * sbyte(bv[q], i);
            }
        }
        uint32_t packed[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            uint32_t wd = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int c = ch + q * 4 + i;
                const int e = p.per_channel ? __ldg(p.ew + c) : p.ew_scalar;
                const int shift = max(-31, min(31, p.e_shift_base - e));
                int32_t v = requant8(acc[q * 4 + i], bias ? __ldg(bias + c) : 0, shift, p.relu, p.half_even);
                if (p.lut)
                    v = p.lut[(uint8_t)v ^ 0x80u];
                wd |= ((uint32_t)v & 0xffu) << (8 * i);
            }
            packed[q] = wd;
        }
        *(uint4 *)(out + pix * p.ops + ch) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
}

template <typename T, typename ACC, typename BIAS>
__global__ void __launch_bounds__(256) dw_generic_kernel(DwParams p)
{
    const T *__restrict__ in = (const T *)p.in;
    const T *__restrict__ w = (const T *)p.w;
    const BIAS *__restrict__ bias = (const BIAS *)p.bias;
    T *__restrict__ out = (T *)p.out;
    for (long long item = blockIdx.x * (long long)blockDim.x + threadIdx.x; item < p.total;
         item += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(item % p.c);
        const long long pix = item / p.c;
        const int ox = (int)(pix % p.ow);
        const int oy = (int)((pix / p.ow) % p.oh);
        const int n = (int)(pix / ((long long)p.ow * p.oh));
        ACC acc = 0;
        for (int ky = 0; ky < p.kh; ky++) {
            const int iy = oy * p.sh + ky * p.dh - p.pt;
            if (iy < 0 || iy >= p.ih)
                continue;
            for (int kx = 0; kx < p.kw; kx++) {
                const int ix = ox * p.sw + kx * p.dw - p.pl;
                if (ix < 0 || ix >= p.iw)
                    continue;
                acc += (ACC)((int)in[(((long long)n * p.ih + iy) * p.iw + ix) * p.ips + c] *
                             (int)w[((long long)ky * p.kw + kx) * p.c + c]);
            }
        }
        const int e = p.per_channel ? p.ew[c] : p.ew_scalar;
        if (sizeof(T) == 1) {
            const int shift = max(-31, min(31, p.e_shift_base - e));
            int32_t v = requant8((int32_t)acc, bias ? (int32_t)bias[c] : 0, shift, p.relu, p.half_even);
            if (p.lut)
                v = p.lut[(uint8_t)v ^ 0x80u];
            out[pix * p.ops + c] = (T)v;
        } else {
            const int shift = max(-62, min(62, p.e_shift_base - e));
            out[pix * p.ops + c] = (T)requant16((long long)acc, bias ? (long long)bias[c] : 0ll, shift, p.relu, p.half_even);
        }
    }
}

int conv2d_depthwise(const espdl_conv_desc &d, cudaStream_t s)
{
    DwParams p;
    p.in = d.input, p.w = d.filter, p.bias = d.bias, p.out = d.output, p.ew = d.filter_exponents, p.lut = d.lut;
    p.n = d.n, p.ih = d.in_h, p.iw = d.in_w, p.c = d.in_c, p.oh = d.out_h, p.ow = d.out_w;
    p.kh = d.kh, p.kw = d.kw, p.sh = d.stride_h, p.sw = d.stride_w, p.dh = d.dilation_h, p.dw = d.dilation_w;
    p.pt = d.pad_top, p.pl = d.pad_left;
    p.ips = d.in_pixel_stride ? d.in_pixel_stride : d.in_c;
    p.ops = d.out_pixel_stride ? d.out_pixel_stride : d.out_c;
    p.e_shift_base = d.out_exponent - d.in_exponent;
    p.ew_scalar = d.filter_exponent, p.per_channel = d.per_channel;
    p.relu = d.activation == ESPDL_ACT_RELU, p.half_even = d.round_mode == ESPDL_ROUND_HALF_EVEN;
    const long long pixels = (long long)d.n * d.out_h * d.out_w;
    const int threads = 256;
    const long long max_blocks = (long long)num_sms() * 32;
    const bool vec = d.dtype == ESPDL_DTYPE_INT8 && d.in_c % 16 == 0 && p.ips % 16 == 0 && p.ops % 16 == 0 &&
        ((uintptr_t)d.input % 16) == 0 && ((uintptr_t)d.output % 16) == 0 && ((uintptr_t)d.filter % 16) == 0;
    if (vec) {
        p.chunks = d.in_c / 16;
        p.total = pixels * p.chunks;
        long long blocks = min((p.total + threads - 1) / threads, max_blocks);
        dw_s8_vec16_kernel<<<(unsigned)blocks, threads, 0, s>>>(p);
    } else {
        p.chunks = 0;
        p.total = pixels * d.in_c;
        long long blocks = min((p.total + threads - 1) / threads, max_blocks);
        if (d.dtype == ESPDL_DTYPE_INT8)
            dw_generic_kernel<int8_t, int32_t, int32_t><<<(unsigned)blocks, threads, 0, s>>>(p);
        else
            dw_generic_kernel<int16_t, long long, long long><<<(unsigned)blocks, threads, 0, s>>>(p);
    }
    count_launch();
    return check_launch("conv2d_depthwise");
}

} // namespace espdl
