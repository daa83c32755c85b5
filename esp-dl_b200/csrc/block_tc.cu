// Fused inverted-residual block: 1x1 expand conv -> 3x3 depthwise conv (stride 1 or 2) -> 1x1 project conv
// (-> residual Add) in ONE launch; the expanded tensor (six times the input in MobileNetV2) never reaches HBM.
// Replaces the reference's chain of dl::module::Conv / Add forwards over dl::base::conv2d<int8_t,...>
// (esp-dl/dl/base/dl_base_conv2d.cpp:9-163), depthwise_conv2d<int8_t,...> (dl_base_depthwise_conv2d.cpp:9-66) and
// elemwise_add (dl_base_add.cpp:8-44), with the same requantisation to int8 after every stage
// (dl_base_activate_buffer.hpp:27-73), so the result is bit-identical to the separate nodes.
//
// A tile is TH x TW output pixels of one image (14x14 at stride 1, 7x7 at stride 2); its input patch
// ((TH-1)S+3) x ((TW-1)S+3) <= 256 pixels is the M dimension of the expand MMAs (halo pixels are recomputed by the
// neighbouring tile).  The hidden channels are walked in chunks of 64; per chunk
//   1. expand:    D1[patch pixel][64]  = X[patch pixel][Cin] . W1[chunk][Cin]^T        tcgen05.mma kind::i8, TMEM
//   2. epilogue1: requantise D1 (bias, shift, ReLU, clamp), zero the pixels outside the image (the depthwise conv's
//                 padding is zero in the hidden tensor), write int8 [row][pixel][64] to shared memory
//   3. depthwise: dp4a over byte-transposed columns of that buffer (a thread owns 4 channels x a band of rows and
//                 walks along x), requantise, write int8 into the 64-byte-swizzled K-major A operand of step 4
//   4. project:   D2[out pixel][Cout] += A2[out pixel][64] . W2[Cout][chunk]^T         accumulates over the chunks
// and after the last chunk epilogue2 requantises D2, adds the residual and stores the tile.
// X (a 4-D TMA box of the NHWC input, zero-filled outside the image), W1 and W2 chunks arrive by TMA; X is
// double-buffered across tiles, everything per chunk is double-buffered across chunks.  Warp roles: TMA producer,
// MMA issuer, 8 epilogue warps (epilogue1 and epilogue2), 8 depthwise warps in two groups that take alternate
// chunks.  expand_filter == NULL: step 1/2 become a copy of the input patch's channels (depthwise -> pointwise pair).
// Every mbarrier wait is bounded (tc::mbar_wait); a wait that expires records ESPDL_ERR_TIMEOUT and all roles leave.
#include "tc_common.cuh"

#include <mutex>

namespace espdl {

__device__ int g_block_tc_error = 0;

int read_and_clear_device_error_block()
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_block_tc_error, sizeof(int)) != cudaSuccess)
        return 0;
    if (v) {
        int zero = 0;
        cudaMemcpyToSymbol(g_block_tc_error, &zero, sizeof(int));
    }
    return v;
}

namespace {

using namespace tc;

constexpr int BK_E_WARPS = 8;
constexpr int BK_DW_WARPS = 8;
constexpr int BK_CTRL_WARPS = 3; // TMA producer, expand MMA issuer, project MMA issuer
constexpr int BK_THREADS = 32 * (BK_CTRL_WARPS + BK_E_WARPS + BK_DW_WARPS);
constexpr int BK_CH = 64;      // hidden channels per chunk
constexpr int BK_PIX = 80;     // bytes between pixels of the hidden buffer: 64 + 16 keeps 128-bit stores of
                               // neighbouring pixels and 32-bit loads of neighbouring rows off each other's banks
constexpr size_t BK_SMEM_LIMIT = 226 * 1024;

enum { X_FULL = 0, X_EMPTY = 2, W1_FULL = 4, W1_EMPTY = 6, D1_FULL = 8, D1_EMPTY = 10, H_FULL = 12, H_EMPTY = 14, A2_FULL = 16, A2_EMPTY = 18,
       W2_FULL = 20, W2_EMPTY = 22, D2_FULL = 24, D2_EMPTY = 25, BK_NBARS = 26 };

struct BlockParams {
    int n, ih, iw, cin, chid, cout, oh, ow, S, pt, pl;
    int TH, TW, PHB, PWB, xtiles, ytiles;
    int mb_in, mb_out, has_expand;
    int kx_swz, kx_blocks, n_chunks;
    int cout_pad, n_split, npiece;
    int hpitch, hrows, nb;
    int tmem_cols, d2_col;
    int off_x, x_bytes, off_w1, w1_bytes, off_w2, w2_bytes, off_h, h_bytes, off_a2, a2_bytes, off_par;
    const int8_t *in;
    int8_t *out;
    const int8_t *res;
    const int8_t *dw_w;
    EpiConfig e1, edw, e2;
    int clip1, clipdw;
};

__device__ __forceinline__ uint32_t lds32(uint32_t a)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory"); }
__device__ __forceinline__ void sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// Offset of the 32-bit word `cq` (4 channels) of row m in the A operand of the project MMA: rows of 64 bytes,
// 16-byte chunk index XOR bits 7..8 of the byte offset (the 64-byte TMA/UMMA swizzle).
__device__ __forceinline__ uint32_t a2_offset(int m, int cq) { return (uint32_t)(m * 64 + ((((cq >> 2) ^ (m >> 1)) & 3) << 4) + (cq & 3) * 4); }

template <int S>
struct BkCol {
    uint32_t t[S == 1 ? 2 : 1][4]; // [row group][channel]: four vertically adjacent pixels of that channel
    uint32_t extra;                // stride 2: the fifth input row, untransposed
};

template <int S>
__device__ __forceinline__ void bk_load_col(BkCol<S> &col, uint32_t addr, int pitch)
{
    constexpr int ROWS_IN = S == 1 ? 6 : 5;
    constexpr int PAIRS = S == 1 ? 3 : 2;
    uint32_t raw[ROWS_IN];
#pragma unroll
    for (int r = 0; r < ROWS_IN; r++) raw[r] = lds32(addr + (uint32_t)(r * pitch));
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
    col.extra = S == 2 ? raw[ROWS_IN - 1] : 0u;
}

// Band of a thread whose channels do not qualify for the one-add-one-shift form (a shift outside 1..24, a huge
// bias, half-even rounding): plain loops with the general requantisation, kept out of line.
__device__ __noinline__ void bk_band_general(const BlockParams &p, uint32_t hid, uint32_t a2, int band, int xb, int xe, int cq, int c0)
{
    const int S = p.S;
    const int rows_out = S == 1 ? 4 : 2;
    for (int ro = 0; ro < rows_out; ro++) {
        const int oyl = band * rows_out + ro;
        if (oyl >= p.TH)
            break;
        for (int x = xb; x < xe; x++) {
            uint32_t wd = 0;
            for (int i = 0; i < 4; i++) {
                const int c = c0 + i;
                int32_t acc = 0;
                for (int ky = 0; ky < 3; ky++)
                    for (int kx = 0; kx < 3; kx++) {
                        const uint32_t a = hid + (uint32_t)((oyl * S + ky) * p.hpitch + (x * S + kx) * BK_PIX + cq * 4);
                        const int v = (int)(int8_t)(lds32(a) >> (8 * i));
                        acc += v * (int)p.dw_w[(ky * 3 + kx) * p.chid + c];
                    }
                const int e = p.edw.per_channel ? p.edw.ew[c] : p.edw.ew_scalar;
                const int shift = max(-31, min(31, p.edw.e_shift_base - e));
                const int q = min(requant8(acc, p.edw.bias ? ((const int32_t *)p.edw.bias)[c] : 0, shift, p.edw.relu, p.edw.half_even), p.clipdw);
                wd |= ((uint32_t)q & 0xffu) << (8 * i);
            }
            sts32(a2 + a2_offset(oyl * p.TW + x, cq), wd);
        }
    }
}

// 3x3 depthwise conv of one band (4 output rows at stride 1, 2 at stride 2) x columns [xb, xe) x 4 channels, from
// the hidden buffer in shared memory into the project MMA's A operand.  dp4a sums four byte products of ONE channel:
// each input column is byte-transposed once (word i = channel i of four vertically adjacent pixels) and multiplied
// with the filter column (w[0][kx], w[1][kx], w[2][kx], 0) and its byte-shifted forms.
template <int S, bool CLIP>
__device__ __forceinline__ void bk_band(const BlockParams &p, uint32_t hid, uint32_t a2, int band, int xb, int xe, int cq, int c0)
{
    constexpr int ROWS_OUT = S == 1 ? 4 : 2;
    uint32_t wv[3][4], wv1[3][4], wsel[3][4];
#pragma unroll
    for (int kx = 0; kx < 3; kx++) {
        uint32_t f[3];
#pragma unroll
        for (int ky = 0; ky < 3; ky++) f[ky] = __ldg((const uint32_t *)(p.dw_w + (ky * 3 + kx) * p.chid + c0));
        const uint32_t lo0 = __byte_perm(f[0], f[1], 0x5140), hi0 = __byte_perm(f[0], f[1], 0x7362);
        const uint32_t lo1 = __byte_perm(f[2], 0u, 0x5140), hi1 = __byte_perm(f[2], 0u, 0x7362);
        wv[kx][0] = __byte_perm(lo0, lo1, 0x5410);
        wv[kx][1] = __byte_perm(lo0, lo1, 0x7632);
        wv[kx][2] = __byte_perm(hi0, hi1, 0x5410);
        wv[kx][3] = __byte_perm(hi0, hi1, 0x7632);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            wv1[kx][i] = wv[kx][i] << (S == 1 ? 8 : 16);             // the band's next output row
            wsel[kx][i] = S == 2 ? (f[2] & (0xffu << (8 * i))) : 0u; // w[2][kx][i] in byte i
        }
    }
    int init[4], shift[4];
    bool fast = !p.edw.half_even;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int b = p.edw.bias ? __ldg((const int32_t *)p.edw.bias + c0 + i) : 0;
        const int e = p.edw.per_channel ? __ldg(p.edw.ew + c0 + i) : p.edw.ew_scalar;
        shift[i] = p.edw.e_shift_base - e;
        // (acc + bias + 2^(s-1)) >> s is exact while nothing can overflow: |acc| <= 9 * 2^14, |bias| < 2^30, 1 <= s <= 24
        fast = fast && shift[i] >= 1 && shift[i] <= 24 && b < (1 << 30) && b > -(1 << 30);
        shift[i] = max(1, min(24, shift[i]));
        init[i] = b + (1 << (shift[i] - 1));
    }
    if (!fast) {
        bk_band_general(p, hid, a2, band, xb, xe, cq, c0);
        return;
    }
    const int floor_q = p.edw.relu ? 0 : INT_MIN;
    const int clip = p.clipdw;
    const int pitch = p.hpitch, tw = p.TW;
    uint32_t hp = hid + (uint32_t)(band * ROWS_OUT * S * pitch + xb * S * BK_PIX + cq * 4);
    int m0 = band * ROWS_OUT * tw + xb;
    const uint32_t a2w = a2 + (uint32_t)((cq & 3) * 4);
    const int chi = cq >> 2;
    bool ovalid[ROWS_OUT];
#pragma unroll
    for (int ro = 0; ro < ROWS_OUT; ro++) ovalid[ro] = band * ROWS_OUT + ro < p.TH;

    auto emit = [&](const BkCol<S> &k0, const BkCol<S> &k1, const BkCol<S> &k2) {
        int acc[ROWS_OUT][4];
#pragma unroll
        for (int kx = 0; kx < 3; kx++) {
            const BkCol<S> &k = kx == 0 ? k0 : (kx == 1 ? k1 : k2);
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
            int q0 = max(acc[ro][0] >> shift[0], floor_q), q1 = max(acc[ro][1] >> shift[1], floor_q);
            int q2 = max(acc[ro][2] >> shift[2], floor_q), q3 = max(acc[ro][3] >> shift[3], floor_q);
            if constexpr (CLIP)
                q0 = min(q0, clip), q1 = min(q1, clip), q2 = min(q2, clip), q3 = min(q3, clip);
            uint32_t hi, wd;
            asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(q3), "r"(q2));
            asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(wd) : "r"(q1), "r"(q0), "r"(hi));
            if (ovalid[ro]) {
                const int m = m0 + ro * tw;
                sts32(a2w + (uint32_t)((m << 6) + (((chi ^ (m >> 1)) & 3) << 4)), wd);
            }
        }
        m0++;
    };

    BkCol<S> ca, cb, cc;
    if constexpr (S == 1) {
        bk_load_col<S>(ca, hp, pitch);
        bk_load_col<S>(cb, hp + BK_PIX, pitch);
        hp += 2 * BK_PIX;
        for (int x = xb; x < xe; x += 3) {
            bk_load_col<S>(cc, hp, pitch);
            emit(ca, cb, cc);
            if (x + 1 >= xe)
                break;
            bk_load_col<S>(ca, hp + BK_PIX, pitch);
            emit(cb, cc, ca);
            if (x + 2 >= xe)
                break;
            bk_load_col<S>(cb, hp + 2 * BK_PIX, pitch);
            emit(cc, ca, cb);
            hp += 3 * BK_PIX;
        }
    } else {
        bk_load_col<S>(ca, hp, pitch);
        hp += BK_PIX;
        for (int x = xb; x < xe; x += 2) {
            bk_load_col<S>(cb, hp, pitch);
            bk_load_col<S>(cc, hp + BK_PIX, pitch);
            emit(ca, cb, cc);
            if (x + 1 >= xe)
                break;
            bk_load_col<S>(cb, hp + 2 * BK_PIX, pitch);
            bk_load_col<S>(ca, hp + 3 * BK_PIX, pitch);
            emit(cc, cb, ca);
            hp += 4 * BK_PIX;
        }
    }
}

// Four accumulator columns -> four saturated int8 with an upper clamp (a folded Clip node).
__device__ __forceinline__ uint32_t requant4_clip(const int32_t *v, uint32_t fp, int floor_q, int clip)
{
    int b0, s0, b1, s1, b2, s2, b3, s3;
    asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(b0), "=r"(s0), "=r"(b1), "=r"(s1) : "r"(fp));
    asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(b2), "=r"(s2), "=r"(b3), "=r"(s3) : "r"(fp + 16));
    const int r0 = min(__viaddmax_s32(v[0], b0, floor_q) >> s0, clip);
    const int r1 = min(__viaddmax_s32(v[1], b1, floor_q) >> s1, clip);
    const int r2 = min(__viaddmax_s32(v[2], b2, floor_q) >> s2, clip);
    const int r3 = min(__viaddmax_s32(v[3], b3, floor_q) >> s3, clip);
    uint32_t hi, w;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(r3), "r"(r2));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(r1), "r"(r0), "r"(hi));
    return w;
}

__device__ __forceinline__ uint32_t clip_bytes(uint32_t w, int clip)
{
    uint32_t r = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) r |= ((uint32_t)min((int)(int8_t)(w >> (8 * i)), clip) & 0xffu) << (8 * i);
    return r;
}

// out = sat(q + r) per byte
__device__ __forceinline__ uint32_t add_bytes_sat(uint32_t q, uint32_t r)
{
    int t[4];
#pragma unroll
    for (int i = 0; i < 4; i++) t[i] = (int)(int8_t)(q >> (8 * i)) + (int)(int8_t)(r >> (8 * i));
    uint32_t hi, w;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(t[3]), "r"(t[2]));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(t[1]), "r"(t[0]), "r"(hi));
    return w;
}

// Bounded wait for the hand-overs of this kernel, which are thousands of cycles apart: the poll carries a suspend-time
// hint, so a waiting warp is parked by the hardware until the phase completes (or the hint runs out) instead of
// spinning through the issue slots that the computing warps need.
__device__ __forceinline__ uint32_t bk_try(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(200000u)
        : "memory");
    return done;
}

__device__ __forceinline__ bool bk_wait(uint32_t bar, uint32_t parity)
{
    if (bk_try(bar, parity))
        return true;
    const long long t0 = clock64();
    while (true) {
#pragma unroll 1
        for (int spin = 0; spin < 64; spin++)
            if (bk_try(bar, parity))
                return true;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES)
            return false;
    }
}

__global__ void __launch_bounds__(BK_THREADS, 1)
block_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w1, const __grid_constant__ CUtensorMap map_w2,
                const __grid_constant__ BlockParams p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const int chid_pad = p.n_chunks * BK_CH;
    FastParam *fp1 = (FastParam *)(smem + p.off_par);
    FastParam *fp2 = fp1 + chid_pad;
    uint64_t *bars = (uint64_t *)(fp2 + p.cout_pad);
    uint32_t *tmem_slot = (uint32_t *)(bars + BK_NBARS);
    int *slow = (int *)(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
#define BAR(i) (bar0 + 8u * (uint32_t)(i))

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_per_image = p.ytiles * p.xtiles;
    const int total_tiles = p.n * tiles_per_image;

    if (threadIdx.x == 0) {
        const int counts[BK_NBARS] = {1, 1, 1, 1, 1, 1, 1, 1, 1, 1, BK_E_WARPS, BK_E_WARPS, BK_E_WARPS, BK_E_WARPS, BK_DW_WARPS / 2, BK_DW_WARPS / 2,
                                      BK_DW_WARPS / 2, BK_DW_WARPS / 2, 1, 1, 1, 1, 1, 1, 1, BK_E_WARPS};
        for (int i = 0; i < BK_NBARS; i++) mbar_init(BAR(i), (uint32_t)counts[i]);
        slow[0] = slow[1] = 0;
        fence_barrier_init();
    }
    if (warp == 1)
        tmem_alloc(smem_u32(tmem_slot), p.tmem_cols);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (p.has_expand)
        stage_fast_params(p.e1, fp1, p.chid, chid_pad, threadIdx.x, BK_THREADS, &slow[0]);
    stage_fast_params(p.e2, fp2, p.cout, p.cout_pad, threadIdx.x, BK_THREADS, &slow[1]);
    __syncthreads();
    const int x_kblock_bytes = 128 * p.mb_in * p.kx_swz;
    const int w1_kblock_bytes = BK_CH * p.kx_swz;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int g = 0, lt = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, lt++) {
                const int img = tile / tiles_per_image;
                const int ty = (tile / p.xtiles) % p.ytiles, tx = tile % p.xtiles;
                if (p.has_expand) {
                    const int tb = lt & 1;
                    if (!bk_wait(BAR(X_EMPTY + tb), ((lt >> 1) & 1) ^ 1)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(BAR(X_FULL + tb), (uint32_t)(p.kx_blocks * p.PWB * p.PHB * p.kx_swz));
                    for (int cb = 0; cb < p.kx_blocks; cb++)
                        tma_load_4d(sbase + p.off_x + tb * p.x_bytes + cb * x_kblock_bytes, &map_x, cb * p.kx_swz, tx * p.TW * p.S - p.pl,
                                    ty * p.TH * p.S - p.pt, img, BAR(X_FULL + tb));
                }
                for (int c = 0; c < p.n_chunks; c++, g++) {
                    const int buf = g & 1;
                    const uint32_t ph = (g >> 1) & 1;
                    if (p.has_expand) {
                        if (!bk_wait(BAR(W1_EMPTY + buf), ph ^ 1)) {
                            ok = false;
                            break;
                        }
                        mbar_arrive_expect_tx(BAR(W1_FULL + buf), (uint32_t)(p.kx_blocks * w1_kblock_bytes));
                        for (int cb = 0; cb < p.kx_blocks; cb++)
                            tma_load_2d(sbase + p.off_w1 + buf * p.w1_bytes + cb * w1_kblock_bytes, &map_w1, cb * p.kx_swz, c * BK_CH, BAR(W1_FULL + buf));
                    }
                    if (!bk_wait(BAR(W2_EMPTY + buf), ph ^ 1)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(BAR(W2_FULL + buf), (uint32_t)(p.n_split * p.npiece * 64));
                    for (int piece = 0; piece < p.n_split; piece++)
                        tma_load_2d(sbase + p.off_w2 + buf * p.w2_bytes + piece * p.npiece * 64, &map_w2, c * BK_CH, piece * p.npiece, BAR(W2_FULL + buf));
                }
            }
            if (!ok)
                atomicExch(&g_block_tc_error, ESPDL_ERR_TIMEOUT);
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ expand MMA issuer
        if (lane == 0 && p.has_expand) {
            int g = 0, lt = 0;
            bool ok = true;
            const uint32_t idesc1 = idesc_i8(1, 1, 128, BK_CH);
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, lt++) {
                const int tb = lt & 1;
                if (!bk_wait(BAR(X_FULL + tb), (lt >> 1) & 1)) {
                    ok = false;
                    break;
                }
                for (int c = 0; c < p.n_chunks; c++, g++) {
                    const int buf = g & 1;
                    const uint32_t ph = (g >> 1) & 1;
                    if (!bk_wait(BAR(W1_FULL + buf), ph) || !bk_wait(BAR(D1_EMPTY + buf), ph ^ 1)) {
                        ok = false;
                        break;
                    }
                    fence_after();
                    for (int mb = 0; mb < p.mb_in; mb++)
                        for (int cb = 0; cb < p.kx_blocks; cb++) {
                            const int ksteps = (min(p.kx_swz, p.cin - cb * p.kx_swz) + 31) / 32;
                            const uint64_t da = smem_desc_swizzled(sbase + p.off_x + tb * p.x_bytes + cb * x_kblock_bytes + mb * 128 * p.kx_swz, p.kx_swz);
                            const uint64_t db = smem_desc_swizzled(sbase + p.off_w1 + buf * p.w1_bytes + cb * w1_kblock_bytes, p.kx_swz);
                            const uint32_t d = tmem_base + (uint32_t)(buf * p.mb_in * BK_CH + mb * BK_CH);
                            for (int k = 0; k < ksteps; k++) mma_i8(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc1, (cb | k) != 0);
                        }
                    commit(BAR(D1_FULL + buf));
                    commit(BAR(W1_EMPTY + buf));
                    if (c == p.n_chunks - 1)
                        commit(BAR(X_EMPTY + tb));
                }
            }
            if (!ok)
                atomicExch(&g_block_tc_error, ESPDL_ERR_TIMEOUT);
        }
        __syncwarp();
    } else if (warp == 2) {
        // ------------------------------------------------------------------ project MMA issuer
        if (lane == 0) {
            int g = 0, lt = 0;
            bool ok = true;
            const uint32_t idesc2 = idesc_i8(1, 1, 128, p.npiece);
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, lt++) {
                for (int c = 0; c < p.n_chunks; c++, g++) {
                    const int buf = g & 1;
                    const uint32_t ph = (g >> 1) & 1;
                    if ((c == 0 && !bk_wait(BAR(D2_EMPTY), (lt & 1) ^ 1)) || !bk_wait(BAR(W2_FULL + buf), ph) || !bk_wait(BAR(A2_FULL + buf), ph)) {
                        ok = false;
                        break;
                    }
                    fence_after();
                    const int ksteps = (min(BK_CH, p.chid - c * BK_CH) + 31) / 32;
                    for (int mb = 0; mb < p.mb_out; mb++)
                        for (int piece = 0; piece < p.n_split; piece++) {
                            const uint64_t da = smem_desc_swizzled(sbase + p.off_a2 + buf * p.a2_bytes + mb * 128 * 64, 64);
                            const uint64_t db = smem_desc_swizzled(sbase + p.off_w2 + buf * p.w2_bytes + piece * p.npiece * 64, 64);
                            const uint32_t d = tmem_base + (uint32_t)(p.d2_col + mb * p.cout_pad + piece * p.npiece);
                            for (int k = 0; k < ksteps; k++) mma_i8(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc2, (c | k) != 0);
                        }
                    commit(BAR(A2_EMPTY + buf));
                    commit(BAR(W2_EMPTY + buf));
                    if (c == p.n_chunks - 1)
                        commit(BAR(D2_FULL));
                }
            }
            if (!ok)
                atomicExch(&g_block_tc_error, ESPDL_ERR_TIMEOUT);
        }
        __syncwarp();
    } else if (warp < BK_CTRL_WARPS + BK_E_WARPS) {
        // ------------------------------------------------------------------ epilogue warps: hidden tensor, then output
        const int e = warp - BK_CTRL_WARPS;
        const int q = e >> 2;      // which half of the work this quad of warps takes
        const int lg = warp & 3;   // TMEM lanes 32*lg .. 32*lg+31 are the ones this warp may read
        const bool fast1 = !slow[0] && !p.e1.half_even && p.cin <= 32768;
        const bool fast2 = !slow[1] && !p.e2.half_even && p.chid <= 32768;
        const uint32_t fp1_base = epi_param_base(fp1);
        const int floor1 = p.e1.relu ? 0 : INT_MIN;
        const uintptr_t amix = (uintptr_t)p.cout | (uintptr_t)p.out | 16u;
        const int out_align = (int)(amix & (~amix + 1));
        const uintptr_t rmix = (uintptr_t)p.cout | (uintptr_t)p.res | 16u;
        const int res_align = (int)(rmix & (~rmix + 1));
        bool ok = true;

        auto epilogue2 = [&](int tile, int tile_lt) -> bool {
            if (!bk_wait(BAR(D2_FULL), tile_lt & 1))
                return false;
            fence_after();
            const int img = tile / tiles_per_image;
            const int ty = (tile / p.xtiles) % p.ytiles, tx = tile % p.xtiles;
            const int mb = p.mb_out == 2 ? q : 0;
            const int m = mb * 128 + lg * 32 + lane;
            const int oyl = m / p.TW, oxl = m % p.TW;
            const int oy = ty * p.TH + oyl, ox = tx * p.TW + oxl;
            const bool row_ok = oyl < p.TH && oy < p.oh && ox < p.ow;
            const long long pix = ((long long)img * p.oh + oy) * p.ow + ox;
            int8_t *orow = p.out + pix * p.cout;
            const int8_t *rrow = p.res ? p.res + pix * p.cout : nullptr;
            const uint32_t t0 = tmem_base + ((uint32_t)(lg * 32) << 16) + (uint32_t)(p.d2_col + mb * p.cout_pad);
            for (int cg = 0; cg * 16 < p.cout_pad; cg++) {
                if (p.mb_out == 1 && (cg & 1) != q)
                    continue;
                int32_t v[16];
                ld16(t0 + cg * 16, v);
                ld_wait16(v);
                uint32_t pk[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                if (fast2) {
                    if (p.e2.relu)
                        requant16_fast<true>(v, fp2 + cg * 16, pk);
                    else
                        requant16_fast<false>(v, fp2 + cg * 16, pk);
                } else {
                    requant16_general(v, p.e2, cg * 16, p.cout, pk);
                }
                const int count = min(16, p.cout - cg * 16);
                if (row_ok && count > 0) {
                    if (rrow) {
                        uint32_t rw[4] = {0, 0, 0, 0};
                        if (count == 16 && res_align >= 16) {
                            const uint4 rr = __ldg((const uint4 *)(rrow + cg * 16));
                            rw[0] = rr.x, rw[1] = rr.y, rw[2] = rr.z, rw[3] = rr.w;
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; j++)
                                if (j < count)
                                    rw[j >> 2] |= (uint32_t)(uint8_t)rrow[cg * 16 + j] << (8 * (j & 3));
                        }
#pragma unroll
                        for (int w = 0; w < 4; w++) pk[w] = add_bytes_sat(pk[w], rw[w]);
                    }
                    store_bytes(orow + cg * 16, pk, count, out_align);
                }
            }
            fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(BAR(D2_EMPTY));
            return true;
        };

        int g = 0, lt = 0, pending_tile = -1;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, lt++) {
            const int img = tile / tiles_per_image;
            const int ty = (tile / p.xtiles) % p.ytiles, tx = tile % p.xtiles;
            const int iy0 = ty * p.TH * p.S - p.pt, ix0 = tx * p.TW * p.S - p.pl;
            for (int c = 0; c < p.n_chunks && ok; c++, g++) {
                const int buf = g & 1;
                const uint32_t ph = (g >> 1) & 1;
                const uint32_t hid = sbase + p.off_h + buf * p.h_bytes;
                if (p.has_expand) {
                    if (!bk_wait(BAR(D1_FULL + buf), ph)) {
                        ok = false;
                        break;
                    }
                    fence_after();
                }
                if (!bk_wait(BAR(H_EMPTY + buf), ph ^ 1)) {
                    ok = false;
                    break;
                }
                if (p.has_expand) {
                    const int mb = p.mb_in == 2 ? q : 0;
                    const int col_begin = p.mb_in == 2 ? 0 : q * 32, col_end = p.mb_in == 2 ? BK_CH : q * 32 + 32;
                    const int pix = mb * 128 + lg * 32 + lane;
                    const int py = pix / p.PWB, px = pix % p.PWB;
                    const bool in_patch = pix < p.PHB * p.PWB;
                    const bool inside = iy0 + py >= 0 && iy0 + py < p.ih && ix0 + px >= 0 && ix0 + px < p.iw;
                    const uint32_t t0 = tmem_base + ((uint32_t)(lg * 32) << 16) + (uint32_t)(buf * p.mb_in * BK_CH + mb * BK_CH);
                    const uint32_t dst = hid + (uint32_t)(py * p.hpitch + px * BK_PIX);
                    // 16 columns at a time into two register sets in turn: the load of the next set is in flight while
                    // this one is requantised
                    auto put16 = [&](int32_t *v, int cc) {
                        uint32_t pk[4];
                        if (fast1) {
                            const uint32_t fpp = fp1_base + (uint32_t)(c * BK_CH + cc) * 8u;
                            if (p.clip1 < 127) {
#pragma unroll
                                for (int w = 0; w < 4; w++) pk[w] = requant4_clip(v + 4 * w, fpp + (uint32_t)(4 * w) * 8u, floor1, p.clip1);
                            } else {
#pragma unroll
                                for (int w = 0; w < 4; w++) pk[w] = requant4_floor(v + 4 * w, fpp + (uint32_t)(4 * w) * 8u, floor1);
                            }
                        } else {
                            requant16_general(v, p.e1, c * BK_CH + cc, p.chid, pk);
                            if (p.clip1 < 127)
#pragma unroll
                                for (int w = 0; w < 4; w++) pk[w] = clip_bytes(pk[w], p.clip1);
                        }
                        if (!inside)
                            pk[0] = pk[1] = pk[2] = pk[3] = 0u; // the depthwise conv pads the HIDDEN tensor with zeros
                        if (in_patch)
                            sts128(dst + (uint32_t)cc, pk[0], pk[1], pk[2], pk[3]);
                    };
                    int32_t va[16], vb[16];
                    ld16(t0 + col_begin, va);
                    ld_wait16(va);
                    for (int cc = col_begin; cc < col_end; cc += 32) {
                        ld16(t0 + cc + 16, vb);
                        put16(va, cc);
                        ld_wait16(vb);
                        const bool more = cc + 32 < col_end;
                        if (more)
                            ld16(t0 + cc + 32, va);
                        put16(vb, cc + 16);
                        if (more)
                            ld_wait16(va);
                    }
                    fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(BAR(D1_EMPTY + buf));
                        mbar_arrive(BAR(H_FULL + buf));
                    }
                } else {
                    // no expand stage: the hidden tensor is the input; copy this chunk's channels of the patch
                    const int pix = e * 32 + lane;
                    const int py = pix / p.PWB, px = pix % p.PWB;
                    if (pix < p.PHB * p.PWB) {
                        const int iy = iy0 + py, ix = ix0 + px;
                        const bool inside = iy >= 0 && iy < p.ih && ix >= 0 && ix < p.iw;
                        const int nbytes = min(BK_CH, p.chid - c * BK_CH);
                        const int8_t *src = p.in + (((long long)img * p.ih + iy) * p.iw + ix) * p.cin + c * BK_CH;
                        const uint32_t dst = hid + (uint32_t)(py * p.hpitch + px * BK_PIX);
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            if (j * 16 < nbytes) {
                                uint4 val = make_uint4(0u, 0u, 0u, 0u);
                                if (inside)
                                    val = __ldg((const uint4 *)(src + j * 16));
                                sts128(dst + (uint32_t)(j * 16), val.x, val.y, val.z, val.w);
                            }
                    }
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(BAR(H_FULL + buf));
                }
                // the previous tile's output epilogue runs one chunk late, so that these warps do not sit waiting
                // for its last depthwise chunk and project MMAs
                if (c == 0 && pending_tile >= 0) {
                    ok = epilogue2(pending_tile, lt - 1);
                    pending_tile = -1;
                }
            }
            pending_tile = tile;
        }
        if (ok && pending_tile >= 0)
            ok = epilogue2(pending_tile, lt - 1);
        if (!ok && lane == 0)
            atomicExch(&g_block_tc_error, ESPDL_ERR_TIMEOUT);
    } else {
        // ------------------------------------------------------------------ depthwise warps
        const int d = warp - BK_CTRL_WARPS - BK_E_WARPS;
        const int grp = d >> 2;
        const int t = (d & 3) * 32 + lane;
        const int cq = t & 15;
        const int band = ((t >> 4) & 1) | (((t >> 6) & 1) << 1);
        const int xh = (t >> 5) & 1;
        const int xm = (p.TW + 1) / 2;
        const int xb = xh ? xm : 0, xe = xh ? p.TW : xm;
        bool ok = true;
        int g = 0;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            for (int c = 0; c < p.n_chunks && ok; c++, g++) {
                if ((g & 1) != grp)
                    continue;
                const uint32_t ph = (g >> 1) & 1;
                if (!bk_wait(BAR(H_FULL + grp), ph) || !bk_wait(BAR(A2_EMPTY + grp), ph ^ 1)) {
                    ok = false;
                    break;
                }
                const int c0 = c * BK_CH + cq * 4;
                if (band < p.nb && c0 < p.chid && xb < xe) {
                    const uint32_t hid = sbase + p.off_h + grp * p.h_bytes;
                    const uint32_t a2 = sbase + p.off_a2 + grp * p.a2_bytes;
                    if (p.clipdw < 127) { // a folded Clip node: rare, kept out of the common path's instruction count
                        if (p.S == 1)
                            bk_band<1, true>(p, hid, a2, band, xb, xe, cq, c0);
                        else
                            bk_band<2, true>(p, hid, a2, band, xb, xe, cq, c0);
                    } else if (p.S == 1) {
                        bk_band<1, false>(p, hid, a2, band, xb, xe, cq, c0);
                    } else {
                        bk_band<2, false>(p, hid, a2, band, xb, xe, cq, c0);
                    }
                }
                fence_async_smem(); // the MMA reads what these threads wrote through the async proxy
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(BAR(A2_FULL + grp));
                    mbar_arrive(BAR(H_EMPTY + grp));
                }
            }
        }
        if (!ok && lane == 0)
            atomicExch(&g_block_tc_error, ESPDL_ERR_TIMEOUT);
    }
#undef BAR

    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        tmem_dealloc(tmem_base, p.tmem_cols);
    }
}


typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn block_encode()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

CUtensorMapSwizzle block_swizzle(int bytes)
{
    return bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

int round_up(int v, int m) { return (v + m - 1) / m * m; }

bool block_plan(const espdl_block_desc &d, BlockParams &p, size_t &smem_bytes, bool check_pointers)
{
    if (d.dtype != ESPDL_DTYPE_INT8 || d.n <= 0 || (d.stride != 1 && d.stride != 2))
        return false;
    if (d.in_c <= 0 || d.hidden_c <= 0 || d.out_c <= 0 || d.out_c > 512 || d.in_c % 16 || d.hidden_c % 16 || d.in_c > 4096 || d.hidden_c > 8192)
        return false;
    if (d.in_h <= 0 || d.in_w <= 0 || d.out_h <= 0 || d.out_w <= 0 || d.pad_top < 0 || d.pad_top > 1 || d.pad_left < 0 || d.pad_left > 1)
        return false;
    if ((d.out_h - 1) * d.stride - d.pad_top >= d.in_h || (d.out_w - 1) * d.stride - d.pad_left >= d.in_w)
        return false;
    if (check_pointers) {
        if (!d.input || !d.output || !d.dw_filter || !d.project_filter || (!d.expand_filter && d.hidden_c != d.in_c))
            return false;
        if (((uintptr_t)d.input % 16) || ((uintptr_t)d.expand_filter % 16) || ((uintptr_t)d.project_filter % 16) || ((uintptr_t)d.dw_filter % 4))
            return false;
    }
    const int acts[3] = {d.expand_activation, d.dw_activation, d.project_activation};
    for (int a : acts)
        if (a != ESPDL_ACT_LINEAR && a != ESPDL_ACT_RELU)
            return false;
    p.n = d.n, p.ih = d.in_h, p.iw = d.in_w, p.cin = d.in_c, p.chid = d.hidden_c, p.cout = d.out_c, p.oh = d.out_h, p.ow = d.out_w;
    p.S = d.stride, p.pt = d.pad_top, p.pl = d.pad_left;
    p.has_expand = d.expand_filter != nullptr || (!check_pointers && d.reserved[0] != 0);
    const int tmax = p.S == 1 ? 14 : 7;
    p.TW = d.out_w < tmax ? d.out_w : tmax, p.TH = d.out_h < tmax ? d.out_h : tmax;
    p.PHB = (p.TH - 1) * p.S + 3, p.PWB = (p.TW - 1) * p.S + 3;
    p.xtiles = (d.out_w + p.TW - 1) / p.TW, p.ytiles = (d.out_h + p.TH - 1) / p.TH;
    p.mb_in = (p.PHB * p.PWB + 127) / 128, p.mb_out = (p.TH * p.TW + 127) / 128;
    p.kx_swz = p.cin >= 96 ? 128 : (p.cin > 32 ? 64 : 32);
    p.kx_blocks = (p.cin + p.kx_swz - 1) / p.kx_swz;
    p.n_chunks = (p.chid + BK_CH - 1) / BK_CH;
    p.n_split = p.cout > 256 ? 2 : 1;
    p.cout_pad = round_up(p.cout, 16 * p.n_split);
    p.npiece = p.cout_pad / p.n_split;
    p.nb = (p.TH + (p.S == 1 ? 4 : 2) - 1) / (p.S == 1 ? 4 : 2);
    if (p.mb_in > 2 || p.mb_out > 2 || p.nb > 4 || p.npiece > 256)
        return false;
    p.hrows = 4 * p.nb + (p.S == 1 ? 2 : 1);
    if (p.hrows < p.PHB)
        p.hrows = p.PHB;
    p.hpitch = 4 * (BK_PIX / 4 * p.PWB + (p.PWB % 2 == 0 ? 4 : 8)); // four rows further lands 16 banks further
    p.d2_col = p.has_expand ? 2 * p.mb_in * BK_CH : 0;
    const int cols = p.d2_col + p.mb_out * p.cout_pad;
    int pow2 = 32;
    while (pow2 < cols) pow2 *= 2;
    if (pow2 > 512)
        return false;
    p.tmem_cols = pow2;
    int off = 0;
    p.off_x = off, p.x_bytes = p.has_expand ? p.kx_blocks * 128 * p.mb_in * p.kx_swz : 0, off += 2 * p.x_bytes;
    p.off_w1 = off, p.w1_bytes = p.has_expand ? round_up(p.kx_blocks * BK_CH * p.kx_swz, 1024) : 0, off += 2 * p.w1_bytes;
    p.off_w2 = off, p.w2_bytes = round_up(p.cout_pad * 64, 1024), off += 2 * p.w2_bytes;
    p.off_a2 = off, p.a2_bytes = p.mb_out * 128 * 64, off += 2 * p.a2_bytes;
    p.off_h = off, p.h_bytes = round_up(p.hrows * p.hpitch, 16), off += 2 * p.h_bytes;
    p.off_par = round_up(off, 16);
    smem_bytes = 1024 + (size_t)p.off_par + sizeof(FastParam) * (size_t)(p.n_chunks * BK_CH + p.cout_pad) + BK_NBARS * 8 + 32;
    return smem_bytes <= BK_SMEM_LIMIT;
}

} // namespace

bool fused_block_supported(const espdl_block_desc &d)
{
    BlockParams p;
    size_t smem;
    return block_plan(d, p, smem, false); // shapes only: the caller may not have buffers yet
}

int fused_block_tc(const espdl_block_desc &d, cudaStream_t s)
{
    BlockParams p;
    size_t smem;
    if (!block_plan(d, p, smem, true))
        return ESPDL_ERR_UNSUPPORTED;
    EncodeTiledFn enc = block_encode();
    if (!enc)
        return set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point not found");
    p.in = (const int8_t *)d.input, p.out = (int8_t *)d.output, p.res = (const int8_t *)d.residual, p.dw_w = (const int8_t *)d.dw_filter;
    const int half_even = d.round_mode == ESPDL_ROUND_HALF_EVEN;
    const int e_hidden = p.has_expand ? d.expand_exponent : d.in_exponent;
    p.e1 = EpiConfig{d.expand_bias, d.expand_filter_exponents, nullptr, d.expand_exponent - d.in_exponent, d.expand_filter_exponent, d.per_channel & 1,
                     d.expand_activation == ESPDL_ACT_RELU, half_even};
    p.edw = EpiConfig{d.dw_bias, d.dw_filter_exponents, nullptr, d.dw_exponent - e_hidden, d.dw_filter_exponent, (d.per_channel >> 1) & 1,
                      d.dw_activation == ESPDL_ACT_RELU, half_even};
    p.e2 = EpiConfig{d.project_bias, d.project_filter_exponents, nullptr, d.out_exponent - d.dw_exponent, d.project_filter_exponent,
                     (d.per_channel >> 2) & 1, d.project_activation == ESPDL_ACT_RELU, half_even};
    p.clip1 = d.expand_clip_max > 127 ? 127 : d.expand_clip_max;
    p.clipdw = d.dw_clip_max > 127 ? 127 : d.dw_clip_max;
    if ((p.e1.per_channel && p.has_expand && !p.e1.ew) || (p.edw.per_channel && !p.edw.ew) || (p.e2.per_channel && !p.e2.ew))
        return set_error_text(ESPDL_ERR_INVALID_ARG, "fused block: per-channel exponents requested without an exponent array");

    CUtensorMap mx, mw1, mw2;
    {
        cuuint64_t dims[2] = {(cuuint64_t)p.chid, (cuuint64_t)p.cout};
        cuuint64_t strides[1] = {(cuuint64_t)p.chid};
        cuuint32_t box[2] = {(cuuint32_t)BK_CH, (cuuint32_t)p.npiece};
        cuuint32_t estr[2] = {1, 1};
        if (enc(&mw2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(d.project_filter), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(block project filter)");
    }
    mx = mw2, mw1 = mw2;
    if (p.has_expand) {
        cuuint64_t dims[4] = {(cuuint64_t)p.cin, (cuuint64_t)p.iw, (cuuint64_t)p.ih, (cuuint64_t)p.n};
        cuuint64_t strides[3] = {(cuuint64_t)p.cin, (cuuint64_t)p.cin * p.iw, (cuuint64_t)p.cin * p.iw * p.ih};
        cuuint32_t box[4] = {(cuuint32_t)p.kx_swz, (cuuint32_t)p.PWB, (cuuint32_t)p.PHB, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        if (enc(&mx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(d.input), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                block_swizzle(p.kx_swz), CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(block input)");
        cuuint64_t wdims[2] = {(cuuint64_t)p.cin, (cuuint64_t)p.chid};
        cuuint64_t wstrides[1] = {(cuuint64_t)p.cin};
        cuuint32_t wbox[2] = {(cuuint32_t)p.kx_swz, (cuuint32_t)BK_CH};
        cuuint32_t westr[2] = {1, 1};
        if (enc(&mw1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(d.expand_filter), wdims, wstrides, wbox, westr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                block_swizzle(p.kx_swz), CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(block expand filter)");
    }
    static std::once_flag attr_once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(attr_once, [] { attr_err = cudaFuncSetAttribute(block_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024); });
    if (attr_err != cudaSuccess)
        return set_cuda_error(attr_err, "cudaFuncSetAttribute(block_tc_kernel)");
    if (smem < 120 * 1024)
        smem = 120 * 1024; // one CTA per SM, so that TMEM allocation never waits on a neighbour
    const long long total = (long long)p.n * p.ytiles * p.xtiles;
    if (total > 0x7fffffffll)
        return ESPDL_ERR_TOO_LARGE;
    const int grid = (int)(total < (long long)num_sms() ? total : (long long)num_sms());
    block_tc_kernel<<<grid, BK_THREADS, smem, s>>>(mx, mw1, mw2, p);
    count_launch();
    return check_launch("block_tc");
}

} // namespace espdl
