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

// 3x3 depthwise, stride S (1 or 2), dilation 1, int8: the workhorse of MobileNet-style networks.
// A thread owns four consecutive channels (one 32-bit word of the NHWC pixel) and a patch of TW x TH output
// pixels.  Its nine filter words, bias and shift stay in registers for the whole patch; input rows slide
// through a three-row register window, so every input word is loaded and unpacked once per patch row; lanes of
// a warp are consecutive channel words of the same pixels, so loads and stores are contiguous runs.
template <int S, int TW, int TH>
__global__ void __launch_bounds__(128) dw3x3_s8_kernel(DwParams p, int xtiles, int ytiles)
{
    constexpr int TWIN = (TW - 1) * S + 3; // input columns feeding TW outputs
    const int quads = p.c >> 2;
    const long long items = (long long)p.n * ytiles * xtiles * quads;
    const long long item = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (item >= items)
        return;
    const int cq = (int)(item % quads);
    long long r = item / quads;
    const int xt = (int)(r % xtiles);
    r /= xtiles;
    const int yt = (int)(r % ytiles);
    const int n = (int)(r / ytiles);
    const int c0 = cq * 4;
    const int8_t *__restrict__ in = (const int8_t *)p.in + (long long)n * p.ih * p.iw * p.ips + c0;
    int8_t *__restrict__ out = (int8_t *)p.out + (long long)n * p.oh * p.ow * p.ops + c0;

    int wt[9][4];
#pragma unroll
    for (int t = 0; t < 9; t++) {
        const uint32_t w = __ldg((const uint32_t *)((const int8_t *)p.w + (long long)t * p.c + c0));
#pragma unroll
        for (int i = 0; i < 4; i++) wt[t][i] = sbyte(w, i);
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
    int bias_half[4];
#pragma unroll
    for (int i = 0; i < 4; i++) bias_half[i] = bias[i] + (1 << (max(1, min(24, shift[i])) - 1));

    const int ox0 = xt * TW, oy0 = yt * TH;
    const int ix0 = ox0 * S - p.pl;
    int win[3][TWIN][4];

    auto load_row = [&](int slot, int iy) {
        const bool row_in = iy >= 0 && iy < p.ih;
        const int8_t *rp = in + ((long long)iy * p.iw + ix0) * p.ips;
#pragma unroll
        for (int x = 0; x < TWIN; x++) {
            const int ix = ix0 + x;
            uint32_t w = 0;
            if (row_in && ix >= 0 && ix < p.iw)
                w = __ldg((const uint32_t *)(rp + (long long)x * p.ips));
#pragma unroll
            for (int i = 0; i < 4; i++) win[slot][x][i] = sbyte(w, i);
        }
    };

    // rows oy0*S - pt + {0, 1} fill the window before the first output row
    load_row(0, oy0 * S - p.pt);
    load_row(1, oy0 * S - p.pt + 1);
#pragma unroll
    for (int ry = 0; ry < TH; ry++) {
        const int oy = oy0 + ry;
        if (oy >= p.oh)
            break;
        // window slots rotate: output row ry reads input rows ry*S + {0,1,2}, held in slots (ry*S + k) % 3
        load_row((ry * S + 2) % 3, oy * S - p.pt + 2);
        if (S == 2 && ry > 0) {
            // stride 2 advanced by two rows: the middle row of this window was not loaded by the previous step
            load_row((ry * S + 1) % 3, oy * S - p.pt + 1);
        }
        int acc[TW][4];
#pragma unroll
        for (int x = 0; x < TW; x++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[x][i] = 0;
#pragma unroll
        for (int ky = 0; ky < 3; ky++)
#pragma unroll
            for (int kx = 0; kx < 3; kx++)
#pragma unroll
                for (int x = 0; x < TW; x++)
#pragma unroll
                    for (int i = 0; i < 4; i++) acc[x][i] += win[(ry * S + ky) % 3][x * S + kx][i] * wt[ky * 3 + kx][i];
#pragma unroll
        for (int x = 0; x < TW; x++) {
            const int ox = ox0 + x;
            if (ox < p.ow) {
                uint32_t wd;
                if (fast) {
                    int q[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        q[i] = (acc[x][i] + bias_half[i]) >> shift[i];
                        if (p.relu)
                            q[i] = max(q[i], 0);
                    }
                    uint32_t hi;
                    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(q[3]), "r"(q[2]));
                    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(wd) : "r"(q[1]), "r"(q[0]), "r"(hi));
                } else {
                    wd = 0;
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        int32_t v = requant8(acc[x][i], bias[i], shift[i], p.relu, p.half_even);
                        if (p.lut)
                            v = p.lut[(uint8_t)v ^ 0x80u];
                        wd |= ((uint32_t)v & 0xffu) << (8 * i);
                    }
                }
                *(uint32_t *)(out + ((long long)oy * p.ow + ox) * p.ops) = wd;
            }
        }
    }
}

// 3x3 depthwise on dp4a, int8, dilation 1, stride S (1 or 2).
// dp4a sums four byte products, but a depthwise filter never sums across channels: the four bytes of a dp4a
// operand have to be four TAPS of one channel.  So a thread (four consecutive channels, one 32-bit word per
// pixel) byte-transposes every group of four horizontally adjacent pixels P0..P3 into one word per channel,
// (P0[c], P1[c], P2[c], P3[c]), with eight PRMTs (two of them shared with the neighbouring group).  Against the
// filter row (w0, w1, w2, 0) that word gives the output centred on P1, against (0, w0, w1, w2) the one centred
// on P2: one dp4a per output, channel and filter row.  Groups step by two pixels (stride 1) so that each yields
// two outputs; with stride 2 groups step by four pixels and the second output of a group takes its third tap
// from the next group ((0,0,w0,w1) here, (w2,0,0,0) there).  Transposed rows stay in registers while the thread
// walks down its column, so every input word is loaded and transposed once per thread.
// Per output that is 3 (S=1) or 4.5 (S=2) dp4a, about one PRMT, one shift and three quarters of a pack,
// instead of nine multiply-adds on unpacked bytes.
template <int S, int NG>
struct DwRow {
    uint32_t t[NG + (S == 2 ? 1 : 0)][4]; // [group][channel] -> four pixels of that channel
};

template <int S, int NG>
__device__ __forceinline__ void dw_load_raw(uint32_t (&raw)[(S == 1 ? 2 : 4) * NG + (S == 1 ? 2 : 4)], const int8_t *__restrict__ in,
                                            int iy, int ix0, int ih, int iw, int ips)
{
    constexpr int NP = (S == 1 ? 2 : 4) * NG + (S == 1 ? 2 : 4);
    constexpr int USED = S == 1 ? NP : NP - 3; // stride 2 reads only the first pixel of its extra group
    const bool row_in = iy >= 0 && iy < ih;
    const int8_t *rp = in + ((long long)iy * iw + ix0) * ips;
#pragma unroll
    for (int x = 0; x < NP; x++) {
        const int ix = ix0 + x;
        raw[x] = 0;
        if (x < USED && row_in && ix >= 0 && ix < iw)
            raw[x] = __ldg((const uint32_t *)(rp + (long long)x * ips));
    }
}

template <int S, int NG>
__device__ __forceinline__ void dw_transpose(DwRow<S, NG> &row, const uint32_t (&raw)[(S == 1 ? 2 : 4) * NG + (S == 1 ? 2 : 4)])
{
    constexpr int NP = (S == 1 ? 2 : 4) * NG + (S == 1 ? 2 : 4);
    uint32_t lo[NP / 2], hi[NP / 2];
#pragma unroll
    for (int j = 0; j < NP / 2; j++) {
        lo[j] = __byte_perm(raw[2 * j], raw[2 * j + 1], 0x5140); // channels 0,1 of the pixel pair, interleaved
        hi[j] = __byte_perm(raw[2 * j], raw[2 * j + 1], 0x7362); // channels 2,3
    }
    constexpr int GROUPS = NG + (S == 2 ? 1 : 0);
    constexpr int PAIR_STEP = S == 1 ? 1 : 2;
#pragma unroll
    for (int g = 0; g < GROUPS; g++) {
        const int a = g * PAIR_STEP, b = a + 1;
        row.t[g][0] = __byte_perm(lo[a], lo[b], 0x5410);
        row.t[g][1] = __byte_perm(lo[a], lo[b], 0x7632);
        row.t[g][2] = __byte_perm(hi[a], hi[b], 0x5410);
        row.t[g][3] = __byte_perm(hi[a], hi[b], 0x7632);
    }
}

template <int S, int NG>
__global__ void __launch_bounds__(128) dw3x3_dp4a_kernel(DwParams p, int xtiles, int ytiles, int rows_per_thread)
{
    constexpr int NP = (S == 1 ? 2 : 4) * NG + (S == 1 ? 2 : 4);
    constexpr int TW = 2 * NG; // outputs per thread and row
    const int quads = p.c >> 2;
    const long long item = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (item >= p.total)
        return;
    const int cq = (int)(item % quads);
    long long r = item / quads;
    const int xt = (int)(r % xtiles);
    r /= xtiles;
    const int yt = (int)(r % ytiles);
    const int n = (int)(r / ytiles);
    const int c0 = cq * 4;
    const int8_t *__restrict__ in = (const int8_t *)p.in + (long long)n * p.ih * p.iw * p.ips + c0;
    int8_t *__restrict__ out = (int8_t *)p.out + (long long)n * p.oh * p.ow * p.ops + c0;

    // filter rows as dp4a operands: wa = (w0,w1,w2,0) per channel and row; the shifted forms are derived from it
    uint32_t wa[3][4];
#pragma unroll
    for (int ky = 0; ky < 3; ky++) {
        uint32_t f[3];
#pragma unroll
        for (int kx = 0; kx < 3; kx++) f[kx] = __ldg((const uint32_t *)((const int8_t *)p.w + (long long)(ky * 3 + kx) * p.c + c0));
        const uint32_t lo0 = __byte_perm(f[0], f[1], 0x5140), hi0 = __byte_perm(f[0], f[1], 0x7362);
        const uint32_t lo1 = __byte_perm(f[2], 0u, 0x5140), hi1 = __byte_perm(f[2], 0u, 0x7362);
        wa[ky][0] = __byte_perm(lo0, lo1, 0x5410);
        wa[ky][1] = __byte_perm(lo0, lo1, 0x7632);
        wa[ky][2] = __byte_perm(hi0, hi1, 0x5410);
        wa[ky][3] = __byte_perm(hi0, hi1, 0x7632);
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
    int init[4]; // what the accumulators start from: bias plus the rounding half on the fast path, else 0
#pragma unroll
    for (int i = 0; i < 4; i++) init[i] = fast ? bias[i] + (1 << (shift[i] - 1)) : 0;

    const int ox0 = xt * TW, oy0 = yt * rows_per_thread;
    const int ix0 = ox0 * S - p.pl;
    const int oy_end = min(p.oh, oy0 + rows_per_thread);

    DwRow<S, NG> ra, rb, rc;
    uint32_t raw[NP], raw2[NP];

    auto emit = [&](const DwRow<S, NG> &r0, const DwRow<S, NG> &r1, const DwRow<S, NG> &r2, int oy) {
#pragma unroll
        for (int g = 0; g < NG; g++) {
            int acc0[4], acc1[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                acc0[i] = init[i];
                acc1[i] = init[i];
            }
#pragma unroll
            for (int ky = 0; ky < 3; ky++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const DwRow<S, NG> &rr = ky == 0 ? r0 : (ky == 1 ? r1 : r2);
                    const uint32_t w = wa[ky][i];
                    acc0[i] = __dp4a((int)rr.t[g][i], (int)w, acc0[i]);
                    if (S == 1) {
                        acc1[i] = __dp4a((int)rr.t[g][i], (int)(w << 8), acc1[i]);
                    } else {
                        acc1[i] = __dp4a((int)rr.t[g][i], (int)(w << 16), acc1[i]);
                        acc1[i] = __dp4a((int)rr.t[g + (S == 2 ? 1 : 0)][i], (int)((w >> 16) & 0xffu), acc1[i]);
                    }
                }
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const int ox = ox0 + 2 * g + half;
                const int *acc = half ? acc1 : acc0;
                if (ox < p.ow) {
                    uint32_t wd;
                    if (fast) {
                        const int q0 = acc[0] >> shift[0], q1 = acc[1] >> shift[1], q2 = acc[2] >> shift[2], q3 = acc[3] >> shift[3];
                        uint32_t hi;
                        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(q3), "r"(q2));
                        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(wd) : "r"(q1), "r"(q0), "r"(hi));
                        if (p.relu)
                            wd = __vmaxs4(wd, 0u);
                    } else {
                        wd = 0;
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            int32_t v = requant8(acc[i], bias[i], shift[i], p.relu, p.half_even);
                            if (p.lut)
                                v = p.lut[(uint8_t)v ^ 0x80u];
                            wd |= ((uint32_t)v & 0xffu) << (8 * i);
                        }
                    }
                    *(uint32_t *)(out + ((long long)oy * p.ow + ox) * p.ops) = wd;
                }
            }
        }
    };

    const int iy0 = oy0 * S - p.pt;
    if (S == 1) {
        // rows iy0, iy0+1 prime the window; each step brings one new row in, already requested one step earlier
        dw_load_raw<S, NG>(raw, in, iy0, ix0, p.ih, p.iw, p.ips);
        dw_transpose<S, NG>(ra, raw);
        dw_load_raw<S, NG>(raw, in, iy0 + 1, ix0, p.ih, p.iw, p.ips);
        dw_transpose<S, NG>(rb, raw);
        dw_load_raw<S, NG>(raw, in, iy0 + 2, ix0, p.ih, p.iw, p.ips);
        for (int oy = oy0; oy < oy_end; oy += 3) {
            dw_transpose<S, NG>(rc, raw);
            dw_load_raw<S, NG>(raw, in, oy + 3 - p.pt, ix0, p.ih, p.iw, p.ips);
            emit(ra, rb, rc, oy);
            if (oy + 1 >= oy_end)
                break;
            dw_transpose<S, NG>(ra, raw);
            dw_load_raw<S, NG>(raw, in, oy + 4 - p.pt, ix0, p.ih, p.iw, p.ips);
            emit(rb, rc, ra, oy + 1);
            if (oy + 2 >= oy_end)
                break;
            dw_transpose<S, NG>(rb, raw);
            dw_load_raw<S, NG>(raw, in, oy + 5 - p.pt, ix0, p.ih, p.iw, p.ips);
            emit(rc, ra, rb, oy + 2);
        }
    } else {
        // output row oy reads input rows 2*oy - pt + {0,1,2}; the last of them is the first of the next output row
        dw_load_raw<S, NG>(raw, in, iy0, ix0, p.ih, p.iw, p.ips);
        dw_transpose<S, NG>(ra, raw);
        dw_load_raw<S, NG>(raw, in, iy0 + 1, ix0, p.ih, p.iw, p.ips);
        dw_load_raw<S, NG>(raw2, in, iy0 + 2, ix0, p.ih, p.iw, p.ips);
        for (int oy = oy0; oy < oy_end; oy += 2) {
            dw_transpose<S, NG>(rb, raw);
            dw_transpose<S, NG>(rc, raw2);
            dw_load_raw<S, NG>(raw, in, 2 * oy + 3 - p.pt, ix0, p.ih, p.iw, p.ips);
            dw_load_raw<S, NG>(raw2, in, 2 * oy + 4 - p.pt, ix0, p.ih, p.iw, p.ips);
            emit(ra, rb, rc, oy);
            if (oy + 1 >= oy_end)
                break;
            dw_transpose<S, NG>(rb, raw);
            dw_transpose<S, NG>(ra, raw2);
            dw_load_raw<S, NG>(raw, in, 2 * oy + 5 - p.pt, ix0, p.ih, p.iw, p.ips);
            dw_load_raw<S, NG>(raw2, in, 2 * oy + 6 - p.pt, ix0, p.ih, p.iw, p.ips);
            emit(rc, rb, ra, oy + 1);
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
    const bool k3 = d.dtype == ESPDL_DTYPE_INT8 && d.kh == 3 && d.kw == 3 && d.dilation_h == 1 && d.dilation_w == 1 &&
        d.stride_h == d.stride_w && (d.stride_h == 1 || d.stride_h == 2) && d.in_c % 4 == 0 && p.ips % 4 == 0 && p.ops % 4 == 0 &&
        ((uintptr_t)d.input % 4) == 0 && ((uintptr_t)d.output % 4) == 0 && ((uintptr_t)d.filter % 4) == 0;
    if (k3) {
        // a thread walks down a whole column of the image when the batch gives enough threads without splitting it
        const int tw = d.stride_h == 1 ? 4 : 2;
        const int xtiles = (d.out_w + tw - 1) / tw;
        const long long per_row_tile = (long long)d.n * xtiles * (d.in_c / 4);
        const long long want = (long long)num_sms() * 4096;
        int rows = d.out_h;
        while (rows > 6 && per_row_tile * ((d.out_h + rows - 1) / rows) < want) rows = (rows + 1) / 2;
        const int ytiles = (d.out_h + rows - 1) / rows;
        const long long items = per_row_tile * ytiles;
        p.total = items, p.chunks = 0;
        const long long blocks = (items + 127) / 128;
        if (blocks > 0x7fffffffll)
            return ESPDL_ERR_TOO_LARGE;
        if (d.stride_h == 1)
            dw3x3_dp4a_kernel<1, 2><<<(unsigned)blocks, 128, 0, s>>>(p, xtiles, ytiles, rows);
        else
            dw3x3_dp4a_kernel<2, 1><<<(unsigned)blocks, 128, 0, s>>>(p, xtiles, ytiles, rows);
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
