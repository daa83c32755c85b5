// The dp4a walk of the 3x3 depthwise kernels over a patch in shared memory (see conv_dw_tma.cu): per-thread filter
// constants, byte-transposed columns, one output column per step.  Shared by the depthwise kernel and by the fused
// depthwise -> pointwise kernel, which differ only in where a result word is stored.
#pragma once
#include "common.cuh"

namespace espdl {
namespace dwt {

// Per-thread constants of the four channels a thread owns: the filter columns as dp4a operands, the accumulator start
// values and the shifts.
template <int S>
struct DwtConsts {
    uint32_t wv[3][4];   // (w[0][kx], w[1][kx], w[2][kx], 0) of channel i
    uint32_t wv1[3][4];  // the same shifted to the band's next output row
    uint32_t wsel[3][4]; // stride 2: w[2][kx] in the byte of its channel
    int init[4], shift[4];
    bool fast;
};

// Where the filter and the requantisation constants of a depthwise conv come from.
struct DwtSource {
    const int8_t *w;          // [3][3][C]
    const int32_t *bias, *ew; // int32[C] or null
    const int8_t *lut;
    int lut_stride; // 0: one table, else entries between the tables of consecutive channels
    int C, e_shift_base, ew_scalar, per_channel, relu, half_even;
};

template <int S>
__device__ __forceinline__ void dwt_load_consts(DwtConsts<S> &k, const DwtSource &p, int c0)
{
#pragma unroll
    for (int kx = 0; kx < 3; kx++) {
        uint32_t f[3];
#pragma unroll
        for (int ky = 0; ky < 3; ky++) f[ky] = __ldg((const uint32_t *)(p.w + (long long)(ky * 3 + kx) * p.C + c0));
        const uint32_t lo0 = __byte_perm(f[0], f[1], 0x5140), hi0 = __byte_perm(f[0], f[1], 0x7362);
        const uint32_t lo1 = __byte_perm(f[2], 0u, 0x5140), hi1 = __byte_perm(f[2], 0u, 0x7362);
        k.wv[kx][0] = __byte_perm(lo0, lo1, 0x5410);
        k.wv[kx][1] = __byte_perm(lo0, lo1, 0x7632);
        k.wv[kx][2] = __byte_perm(hi0, hi1, 0x5410);
        k.wv[kx][3] = __byte_perm(hi0, hi1, 0x7632);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            k.wv1[kx][i] = k.wv[kx][i] << (S == 1 ? 8 : 16);
            k.wsel[kx][i] = S == 2 ? (f[2] & (0xffu << (8 * i))) : 0u;
        }
    }
    k.fast = !p.half_even && !p.lut;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int b = p.bias ? __ldg(p.bias + c0 + i) : 0;
        const int e = p.per_channel ? __ldg(p.ew + c0 + i) : p.ew_scalar;
        const int s = max(-31, min(31, p.e_shift_base - e));
        // (acc + bias + 2^(s-1)) >> s is exact while nothing can overflow: |acc| <= 9 * 2^14, |bias| < 2^30, 1 <= s <= 24
        k.fast = k.fast && s >= 1 && s <= 24 && b < (1 << 30) && b > -(1 << 30);
        k.shift[i] = s - (p.relu ? 1 : 0); // what the walk shifts by (see dwt_emit); the general form recomputes its own
        k.init[i] = b + (s >= 1 ? (1 << (s - 1)) : 0);
    }
}

// Four (stride 1) or two (stride 2) vertically adjacent pixels per channel in one word, from the raw rows of a column.
template <int S>
struct DwtCol {
    uint32_t t[S == 1 ? 2 : 1][4];
    uint32_t extra; // stride 2: the fifth input row, untransposed
};

template <int S>
__device__ __forceinline__ void dwt_transpose(DwtCol<S> &col, const uint32_t (&raw)[S == 1 ? 6 : 5])
{
    constexpr int PAIRS = S == 1 ? 3 : 2;
    uint32_t lo[PAIRS], hi[PAIRS];
#pragma unroll
    for (int j = 0; j < PAIRS; j++) {
        lo[j] = __byte_perm(raw[2 * j], raw[2 * j + 1], 0x5140);
        hi[j] = __byte_perm(raw[2 * j], raw[2 * j + 1], 0x7362);
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

// One output column of a band (ROWS_OUT pixels x four channels) from three transposed input columns.
// `st(ro, x, word)` stores the four channels of output row `ro` of the band at column `x` of the run.
template <int S, typename Store>
__device__ __forceinline__ void dwt_emit(const DwtConsts<S> &k, const DwtCol<S> &k0, const DwtCol<S> &k1, const DwtCol<S> &k2, const Store &st, int x, int floor_q)
{
    constexpr int ROWS_OUT = S == 1 ? 4 : 2;
    int acc[ROWS_OUT][4];
#pragma unroll
    for (int kx = 0; kx < 3; kx++) {
        const DwtCol<S> &c = kx == 0 ? k0 : (kx == 1 ? k1 : k2);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t w = k.wv[kx][i], w1 = k.wv1[kx][i];
            if constexpr (S == 1) {
                acc[0][i] = __dp4a((int)c.t[0][i], (int)w, kx == 0 ? k.init[i] : acc[0][i]);
                acc[1][i] = __dp4a((int)c.t[0][i], (int)w1, kx == 0 ? k.init[i] : acc[1][i]);
                acc[2][i] = __dp4a((int)c.t[1][i], (int)w, kx == 0 ? k.init[i] : acc[2][i]);
                acc[3][i] = __dp4a((int)c.t[1][i], (int)w1, kx == 0 ? k.init[i] : acc[3][i]);
            } else {
                acc[0][i] = __dp4a((int)c.t[0][i], (int)w, kx == 0 ? k.init[i] : acc[0][i]);
                acc[1][i] = __dp4a((int)c.t[0][i], (int)w1, kx == 0 ? k.init[i] : acc[1][i]);
                acc[1][i] = __dp4a((int)c.extra, (int)k.wsel[kx][i], acc[1][i]);
            }
        }
    }
    if (floor_q == 0) {
        // ReLU: the staged shifts are one less than the real ones; packing with saturation to [0, 255] clamps below at
        // zero, halving every byte completes the shift and turns the upper clamp into 127 - a shift and a mask per
        // word instead of a max per output
#pragma unroll
        for (int ro = 0; ro < ROWS_OUT; ro++) {
            const int q0 = acc[ro][0] >> k.shift[0], q1 = acc[ro][1] >> k.shift[1], q2 = acc[ro][2] >> k.shift[2], q3 = acc[ro][3] >> k.shift[3];
            uint32_t hi, wd;
            asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(q3), "r"(q2));
            asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(wd) : "r"(q1), "r"(q0), "r"(hi));
            st(ro, x, (wd >> 1) & 0x7f7f7f7fu);
        }
    } else {
#pragma unroll
        for (int ro = 0; ro < ROWS_OUT; ro++) {
            const int q0 = acc[ro][0] >> k.shift[0], q1 = acc[ro][1] >> k.shift[1], q2 = acc[ro][2] >> k.shift[2], q3 = acc[ro][3] >> k.shift[3];
            uint32_t hi, wd;
            asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(q3), "r"(q2));
            asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(wd) : "r"(q1), "r"(q0), "r"(hi));
            st(ro, x, wd);
        }
    }
}

// The run of one thread: L output columns of its band, four channels.  `ip` points at the thread's word in the
// patch's first row and column of the run; results go through `st` (see dwt_emit).  CB4 = channel-block width in words:
// a template argument where the launch has one (column steps become immediate offsets), else `cb4`.
template <int S, int CB4T, typename Store>
__device__ __forceinline__ void dwt_walk(const DwtConsts<S> &k, const uint32_t *ip, const Store &st, int in_row_words, int cb4, int L, int floor_q)
{
    constexpr int ROWS_IN = S == 1 ? 6 : 5;
    const int CB4 = CB4T ? CB4T : cb4;
    const uint32_t *rp[ROWS_IN];
#pragma unroll
    for (int r = 0; r < ROWS_IN; r++) rp[r] = ip + r * in_row_words;
    uint32_t raw[ROWS_IN];
    auto load_col = [&](int j) {
#pragma unroll
        for (int r = 0; r < ROWS_IN; r++) raw[r] = rp[r][j * CB4];
    };
    auto advance = [&](int cols) {
#pragma unroll
        for (int r = 0; r < ROWS_IN; r++) rp[r] += cols * CB4;
    };
    DwtCol<S> ca, cb, cc;
    if constexpr (S == 1) {
        // output x reads input columns x + {0,1,2}: two columns prime the window, every step brings one in
        load_col(0);
        dwt_transpose<S>(ca, raw);
        load_col(1);
        dwt_transpose<S>(cb, raw);
        load_col(2);
        for (int x = 0; x < L; x += 3) {
            dwt_transpose<S>(cc, raw);
            load_col(3);
            dwt_emit<S>(k, ca, cb, cc, st, x, floor_q);
            if (x + 1 >= L)
                break;
            dwt_transpose<S>(ca, raw);
            load_col(4);
            dwt_emit<S>(k, cb, cc, ca, st, x + 1, floor_q);
            if (x + 2 >= L)
                break;
            dwt_transpose<S>(cb, raw);
            load_col(5);
            dwt_emit<S>(k, cc, ca, cb, st, x + 2, floor_q);
            advance(3);
        }
    } else {
        // output x reads input columns 2x + {0,1,2}; the last of them is the first of the next output
        load_col(0);
        dwt_transpose<S>(ca, raw);
        for (int x = 0; x < L; x += 2) {
            load_col(1);
            dwt_transpose<S>(cb, raw);
            load_col(2);
            dwt_transpose<S>(cc, raw);
            dwt_emit<S>(k, ca, cb, cc, st, x, floor_q);
            if (x + 1 >= L)
                break;
            load_col(3);
            dwt_transpose<S>(cb, raw);
            load_col(4);
            dwt_transpose<S>(ca, raw);
            dwt_emit<S>(k, cc, cb, ca, st, x + 1, floor_q);
            advance(4);
        }
    }
}

} // namespace dwt
} // namespace espdl
