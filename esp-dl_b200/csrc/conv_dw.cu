// DepthwiseConv2D (group == channels), int8 and int16.
// Replaces dl::base::depthwise_conv2d<> (esp-dl/dl/base/dl_base_depthwise_conv2d.cpp:47-66,
// shell esp-dl/dl/base/dl_base.hpp:1209-2107): out[y,x,c] = epilogue(sum_{ky,kx} in[..,c] * w[ky,kx,c] + bias[c]).
//
// The op is bandwidth bound by design (9 MACs per byte read).  3x3 filters with stride 1 or 2 - the shapes of
// MobileNet-style networks - run on dw3x3_dp4a_kernel (a thread walks along a band of rows, dp4a over byte-transposed
// columns); other int8 shapes with C % 16 == 0 on dw_s8_vec16_kernel (16 channels per thread, 128-bit loads and
// stores, a warp reads and writes contiguous runs of the NHWC tensor); everything else on dw_generic_kernel.
#include "common.cuh"

namespace espdl {

struct DwParams {
    const void *in, *w, *bias;
    void *out;
    const int32_t *ew;
    const int8_t *lut;
    int lut_stride; // 0: one table, else entries between the tables of consecutive channels
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
                    v = p.lut[(long long)c * p.lut_stride + ((uint8_t)v ^ 0x80u)];
                wd |= ((uint32_t)v & 0xffu) << (8 * i);
            }
            packed[q] = wd;
        }
        *(uint4 *)(out + pix * p.ops + ch) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
}

// 3x3 depthwise on dp4a, int8, dilation 1, stride S (1 or 2).
// dp4a sums four byte products, but a depthwise filter never sums across channels: the four bytes of a dp4a
// operand have to be four TAPS of one channel.  A thread owns four consecutive channels (one 32-bit word of an
// NHWC pixel) and a band of output rows, and walks along the row.  Each input column it meets (the band's input
// rows at one x) is byte-transposed once, eight PRMTs per four rows: word i of a group holds channel i of four
// vertically adjacent pixels.  Against the filter column (w[0][kx], w[1][kx], w[2][kx], 0) that word gives the
// output row whose window starts at the group's first row, against the same word shifted by one byte the next
// row (stride 1, two overlapping groups per band -> four output rows from six input rows).  With stride 2 the
// second output row of a band takes two taps from the group ((0,0,w0,w1)) and its third from a fifth input row,
// read untransposed with the tap placed in the byte of its channel.  Three transposed columns are live; per
// output that is 3 (S=1) or 4.5 (S=2) dp4a, about one PRMT, a shift, a max and half a pack.
// Rows outside the image walk along a row of zeros instead (g_dw_zero_row), so the walk has no per-load bounds
// checks and one step size; columns outside the image are skipped as a whole.  Three columns are always in flight
// (stride 1): with 16 warps per SM it is the bytes in flight, not the arithmetic, that set the speed.
constexpr int DW_ZERO_ROW_BYTES = 128 * 1024;
__device__ uint32_t g_dw_zero_row[DW_ZERO_ROW_BYTES / 4]; // never written: what rows outside the image read

template <int S>
struct DwCol {
    uint32_t t[S == 1 ? 2 : 1][4]; // [row group][channel]: four vertically adjacent pixels of that channel
    uint32_t extra;                // stride 2: the fifth input row, untransposed
};

template <int S>
__device__ __forceinline__ void dw_transpose_col(DwCol<S> &col, const uint32_t (&raw)[S == 1 ? 6 : 5])
{
    constexpr int PAIRS = S == 1 ? 3 : 2;
    uint32_t lo[PAIRS], hi[PAIRS];
#pragma unroll
    for (int j = 0; j < PAIRS; j++) {
        lo[j] = __byte_perm(raw[2 * j], raw[2 * j + 1], 0x5140); // channels 0,1 of the row pair, interleaved
        hi[j] = __byte_perm(raw[2 * j], raw[2 * j + 1], 0x7362); // channels 2,3
    }
#pragma unroll
    for (int g = 0; g < (S == 1 ? 2 : 1); g++) {
        col.t[g][0] = __byte_perm(lo[g], lo[g + 1], 0x5410);
        col.t[g][1] = __byte_perm(lo[g], lo[g + 1], 0x7632);
        col.t[g][2] = __byte_perm(hi[g], hi[g + 1], 0x5410);
        col.t[g][3] = __byte_perm(hi[g], hi[g + 1], 0x7632);
    }
    col.extra = S == 2 ? raw[S == 2 ? 4 : 0] : 0u;
}

// Band of a thread whose channels do not qualify for the one-add-one-shift epilogue (a shift outside 1..24, a
// huge bias, half-even rounding or a fused table): plain loops with the general requantisation.  Kept out of line
// so that the walk below carries none of its registers.
__device__ __noinline__ void dw3x3_band_general(const DwParams &p, int S, int n, int c0, int oy0, int rows, int x_begin, int x_end)
{
    const int8_t *__restrict__ in = (const int8_t *)p.in + (long long)n * p.ih * p.iw * p.ips;
    int8_t *__restrict__ out = (int8_t *)p.out + (long long)n * p.oh * p.ow * p.ops;
    for (int oy = oy0; oy < min(p.oh, oy0 + rows); oy++)
        for (int ox = x_begin; ox < x_end; ox++)
            for (int i = 0; i < 4; i++) {
                const int c = c0 + i;
                int32_t acc = 0;
                for (int ky = 0; ky < 3; ky++)
                    for (int kx = 0; kx < 3; kx++) {
                        const int iy = oy * S - p.pt + ky, ix = ox * S - p.pl + kx;
                        if (iy >= 0 && iy < p.ih && ix >= 0 && ix < p.iw)
                            acc += (int)in[((long long)iy * p.iw + ix) * p.ips + c] * (int)((const int8_t *)p.w)[(ky * 3 + kx) * p.c + c];
                    }
                const int e = p.per_channel ? p.ew[c] : p.ew_scalar;
                const int shift = max(-31, min(31, p.e_shift_base - e));
                int32_t v = requant8(acc, p.bias ? ((const int32_t *)p.bias)[c] : 0, shift, p.relu, p.half_even);
                if (p.lut)
                    v = p.lut[(long long)c * p.lut_stride + ((uint8_t)v ^ 0x80u)];
                out[((long long)oy * p.ow + ox) * p.ops + c] = (int8_t)v;
            }
}

template <int S>
__global__ void __launch_bounds__(128, 4) dw3x3_dp4a_kernel(DwParams p, int xsegs, int ytiles, int cols_per_thread)
{
    constexpr int ROWS_IN = S == 1 ? 6 : 5;
    constexpr int ROWS_OUT = S == 1 ? 4 : 2;
    const int quads = p.c >> 2;
    const long long item = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (item >= p.total)
        return;
    const int cq = (int)(item % quads);
    long long r = item / quads;
    const int yt = (int)(r % ytiles);
    r /= ytiles;
    const int xs = (int)(r % xsegs);
    const int n = (int)(r / xsegs);
    const int c0 = cq * 4;

    // filter columns as dp4a operands: wv[kx][i] = (w[0][kx][i], w[1][kx][i], w[2][kx][i], 0)
    uint32_t wv[3][4], wv1[3][4], wsel[3][4];
#pragma unroll
    for (int kx = 0; kx < 3; kx++) {
        uint32_t f[3];
#pragma unroll
        for (int ky = 0; ky < 3; ky++) f[ky] = __ldg((const uint32_t *)((const int8_t *)p.w + (long long)(ky * 3 + kx) * p.c + c0));
        const uint32_t lo0 = __byte_perm(f[0], f[1], 0x5140), hi0 = __byte_perm(f[0], f[1], 0x7362);
        const uint32_t lo1 = __byte_perm(f[2], 0u, 0x5140), hi1 = __byte_perm(f[2], 0u, 0x7362);
        wv[kx][0] = __byte_perm(lo0, lo1, 0x5410);
        wv[kx][1] = __byte_perm(lo0, lo1, 0x7632);
        wv[kx][2] = __byte_perm(hi0, hi1, 0x5410);
        wv[kx][3] = __byte_perm(hi0, hi1, 0x7632);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            wv1[kx][i] = wv[kx][i] << (S == 1 ? 8 : 16);                           // the band's next output row
            wsel[kx][i] = S == 2 ? (f[2] & (0xffu << (8 * i))) : 0u;               // w[2][kx][i] in byte i
        }
    }
    int bias[4], shift[4];
    bool fast = !p.half_even && !p.lut;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        bias[i] = p.bias ? __ldg((const int32_t *)p.bias + c0 + i) : 0;
        const int e = p.per_channel ? __ldg(p.ew + c0 + i) : p.ew_scalar;
        shift[i] = max(-31, min(31, p.e_shift_base - e));
        // (acc + bias + 2^(s-1)) >> s is exact while nothing can overflow: |acc| <= 9 * 2^14, |bias| < 2^30, 1 <= s <= 24
        fast = fast && shift[i] >= 1 && shift[i] <= 24 && bias[i] < (1 << 30) && bias[i] > -(1 << 30);
    }
    const int oy0 = yt * ROWS_OUT;
    const int x_begin = xs * cols_per_thread, x_end = min(p.ow, x_begin + cols_per_thread);
    if (!fast) {
        dw3x3_band_general(p, S, n, c0, oy0, ROWS_OUT, x_begin, x_end);
        return;
    }
    int init[4]; // accumulators start from bias plus the rounding half
#pragma unroll
    for (int i = 0; i < 4; i++) init[i] = bias[i] + (1 << (shift[i] - 1));
    const int floor_q = p.relu ? 0 : INT_MIN;
    const int iy0 = oy0 * S - p.pt;
    int ix = x_begin * S - p.pl; // column the row pointers stand on

    // one pointer per input row of the band; rows outside the image walk along the row of zeros
    const int8_t *rp[ROWS_IN];
    {
        const int8_t *img = (const int8_t *)p.in + (long long)n * p.ih * p.iw * p.ips + c0;
#pragma unroll
        for (int rr = 0; rr < ROWS_IN; rr++) {
            const int iy = iy0 + rr;
            const bool ok = iy >= 0 && iy < p.ih;
            rp[rr] = ok ? img + ((long long)iy * p.iw + ix) * p.ips : (const int8_t *)g_dw_zero_row + (long long)(ix + 2) * p.ips;
        }
    }
    int8_t *op = (int8_t *)p.out + (((long long)n * p.oh + oy0) * p.ow + x_begin) * p.ops + c0;
    const int orow = p.ow * p.ops;
    bool ovalid[ROWS_OUT];
#pragma unroll
    for (int ro = 0; ro < ROWS_OUT; ro++) ovalid[ro] = oy0 + ro < p.oh;

    uint32_t raw[ROWS_IN], raw2[ROWS_IN], raw3[ROWS_IN], raw4[ROWS_IN];
    auto load_col = [&](uint32_t (&dst)[ROWS_IN]) {
        const bool ok = ix >= 0 && ix < p.iw;
#pragma unroll
        for (int rr = 0; rr < ROWS_IN; rr++) {
            dst[rr] = ok ? __ldg((const uint32_t *)rp[rr]) : 0u;
            rp[rr] += p.ips;
        }
        ix++;
    };

    auto emit = [&](const DwCol<S> &k0, const DwCol<S> &k1, const DwCol<S> &k2) {
        int acc[ROWS_OUT][4];
#pragma unroll
        for (int kx = 0; kx < 3; kx++) {
            const DwCol<S> &k = kx == 0 ? k0 : (kx == 1 ? k1 : k2);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t w = wv[kx][i], w1 = wv1[kx][i];
                if constexpr (S == 1) {
                    acc[0][i] = __dp4a((int)k.t[0][i], (int)w, kx == 0 ? init[i] : acc[0][i]);
                    acc[1][i] = __dp4a((int)k.t[0][i], (int)w1, kx == 0 ? init[i] : acc[1][i]);
                    acc[2][i] = __dp4a((int)k.t[1][i], (int)w, kx == 0 ? init[i] : acc[2][i]);
                    acc[3][i] = __dp4a((int)k.t[1][i], (int)w1, kx == 0 ? init[i] : acc[3][i]);
                } else {
                    acc[0][i] = __dp4a((int)k.t[0][i], (int)w, kx == 0 ? init[i] : acc[0][i]);
                    acc[1][i] = __dp4a((int)k.t[0][i], (int)w1, kx == 0 ? init[i] : acc[1][i]);
                    acc[1][i] = __dp4a((int)k.extra, (int)wsel[kx][i], acc[1][i]);
                }
            }
        }
#pragma unroll
        for (int ro = 0; ro < ROWS_OUT; ro++) {
            const int q0 = max(acc[ro][0] >> shift[0], floor_q), q1 = max(acc[ro][1] >> shift[1], floor_q);
            const int q2 = max(acc[ro][2] >> shift[2], floor_q), q3 = max(acc[ro][3] >> shift[3], floor_q);
            uint32_t hi, wd;
            asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(q3), "r"(q2));
            asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(wd) : "r"(q1), "r"(q0), "r"(hi));
            if (ovalid[ro])
                *(uint32_t *)(op + (long long)ro * orow) = wd;
        }
        op += p.ops;
    };

    DwCol<S> ca, cb, cc;
    if constexpr (S == 1) {
        // output x reads input columns x - pl + {0,1,2}: two columns prime the window, every step brings one in,
        // requested one step before it is needed
        load_col(raw);
        dw_transpose_col<S>(ca, raw);
        load_col(raw);
        dw_transpose_col<S>(cb, raw);
        load_col(raw);
        load_col(raw2);
        load_col(raw3);
        // three column registers and three load buffers rotate together: the pattern repeats every three outputs
        for (int x = x_begin; x < x_end; x += 3) {
            dw_transpose_col<S>(cc, raw);
            load_col(raw);
            emit(ca, cb, cc);
            if (x + 1 >= x_end)
                break;
            dw_transpose_col<S>(ca, raw2);
            load_col(raw2);
            emit(cb, cc, ca);
            if (x + 2 >= x_end)
                break;
            dw_transpose_col<S>(cb, raw3);
            load_col(raw3);
            emit(cc, ca, cb);
        }
    } else {
        // output x reads input columns 2x - pl + {0,1,2}; the last of them is the first of the next output
        load_col(raw);
        dw_transpose_col<S>(ca, raw);
        load_col(raw);
        load_col(raw2);
        load_col(raw3);
        load_col(raw4);
        // two pairs of load buffers alternate, so four columns are in flight
        for (int x = x_begin; x < x_end; x += 2) {
            dw_transpose_col<S>(cb, raw);
            dw_transpose_col<S>(cc, raw2);
            load_col(raw);
            load_col(raw2);
            emit(ca, cb, cc);
            if (x + 1 >= x_end)
                break;
            dw_transpose_col<S>(cb, raw3);
            dw_transpose_col<S>(ca, raw4);
            load_col(raw3);
            load_col(raw4);
            emit(cc, cb, ca);
        }
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
                v = p.lut[(long long)c * p.lut_stride + ((uint8_t)v ^ 0x80u)];
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
    p.in = d.input, p.w = d.filter, p.bias = d.bias, p.out = d.output, p.ew = d.filter_exponents, p.lut = d.lut, p.lut_stride = d.lut_channel_stride;
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
    const bool k3 = d.dtype == ESPDL_DTYPE_INT8 && d.kh == 3 && d.kw == 3 && d.dilation_h == 1 && d.dilation_w == 1 &&
        d.stride_h == d.stride_w && (d.stride_h == 1 || d.stride_h == 2) && d.in_c % 4 == 0 && p.ips % 4 == 0 && p.ops % 4 == 0 &&
        ((uintptr_t)d.input % 4) == 0 && ((uintptr_t)d.output % 4) == 0 && ((uintptr_t)d.filter % 4) == 0;
    if (k3 && ((long long)d.in_w + 10) * p.ips <= DW_ZERO_ROW_BYTES) {
        // a thread walks along a whole band of rows when the batch gives enough threads without cutting the band
        const int rows_out = d.stride_h == 1 ? 4 : 2;
        const int ytiles = (d.out_h + rows_out - 1) / rows_out;
        const long long per_seg = (long long)d.n * ytiles * (d.in_c / 4);
        const long long want = (long long)num_sms() * 2048;
        int cols = d.out_w;
        while (cols > 8 && per_seg * ((d.out_w + cols - 1) / cols) < want) cols = (cols + 1) / 2;
        const int xsegs = (d.out_w + cols - 1) / cols;
        const long long items = per_seg * xsegs;
        p.total = items, p.chunks = 0;
        const long long blocks = (items + 127) / 128;
        if (blocks > 0x7fffffffll)
            return ESPDL_ERR_TOO_LARGE;
        if (d.stride_h == 1)
            dw3x3_dp4a_kernel<1><<<(unsigned)blocks, 128, 0, s>>>(p, xsegs, ytiles, cols);
        else
            dw3x3_dp4a_kernel<2><<<(unsigned)blocks, 128, 0, s>>>(p, xsegs, ytiles, cols);
    } else if (vec) {
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
