// Fused 3x3 depthwise conv -> pointwise conv (-> residual Add), int8: the "depthwise feeds pointwise" pair of an
// inverted-residual block in ONE launch, the tensor between the two never leaving the SM.
//
// Replaces the node chain Conv(group = C, 3x3) -> Conv(1x1) [-> Add] of the reference
// (esp-dl/dl/module/include/dl_module_conv.hpp:121-162, dl_module_add.hpp:43-82; kernels
// esp-dl/dl/base/dl_base_depthwise_conv2d.cpp:47-66 and dl_base_conv2d.cpp:9-60, epilogue
// esp-dl/dl/base/dl_base_activate_buffer.hpp:27-73): the depthwise result is requantised, clamped and saturated to int8
// exactly as the separate node would write it, and that int8 value is what the pointwise product reads.
//
// One persistent CTA per SM, 18 warps:
//   warp 0      producer: per step (one tile x one block of CB hidden channels) a 4-D TMA box with the input patch
//               (zero-filled outside the image) and a 2-D box with the CB columns of the pointwise filter, each into a
//               two-stage ring;
//   warps 6-17  depthwise: a thread owns four channels, a band of output rows and a run of L output columns of the
//               tile (fixed for the launch) and walks it with dp4a over byte-transposed columns (dw_walk.cuh); the
//               requantised words go straight into the A operand of the pointwise MMA in shared memory - rows are
//               output pixels, K-major, in the swizzle the tensor cores read;
//   warp 1      one thread issues tcgen05.mma kind::i8 (M = 128 pixels, N = output channels, K = 32 per instruction),
//               accumulating over the channel blocks of the tile in TMEM;
//   warps 2-5   epilogue: TMEM -> bias, shift, round, (ReLU), saturate -> optional saturating Add of the residual
//               -> NHWC rows in global memory.
// HBM sees the block's input once and its output once; the hidden tensor after the depthwise conv (as large as the
// input) is never written or read back.  Every mbarrier wait is bounded; on expiry the CTA notes ESPDL_ERR_TIMEOUT and
// all roles run their loops to the end without touching memory they do not own, so that no barrier is left unmatched.
#include "dw_walk.cuh"
#include "tc_common.cuh"

#include <cmath>
#include <cstdio>
#include <map>
#include <mutex>
#include <tuple>

namespace espdl {

__device__ int g_dwpw_error = 0;

int read_and_clear_device_error_dwpw()
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_dwpw_error, sizeof(int)) != cudaSuccess)
        return 0;
    if (v) {
        int zero = 0;
        cudaMemcpyToSymbol(g_dwpw_error, &zero, sizeof(int));
    }
    return v;
}

namespace {

using namespace tc;
using namespace dwt;

constexpr int DP_DW_WARPS = 12;
constexpr int DP_DW_THREADS = DP_DW_WARPS * 32;
constexpr int DP_FIRST_DW_WARP = 6;
constexpr int DP_THREADS = (DP_FIRST_DW_WARP + DP_DW_WARPS) * 32;
constexpr int DP_STAGES = 2;
constexpr size_t DP_SMEM_BUDGET = 210 * 1024;

struct DpParams {
    int S, CB, pitch, ksteps;                  // channel block, bytes per row of the A / filter operands (the swizzle width), MMAs per block
    int NB, TH, TW, IH, IW, L, nseg, nbands, items;
    int MB, m_valid;                           // 128-row blocks per tile, pixels of a tile
    int cblocks, nblocks, ytiles, xtiles, total_tiles;
    int N, OH, OW, cout, n_pad, tmem_cols;
    int pt, pl;
    int patch_bytes, patch_tx, w2_bytes, w2_tx, a_bytes; // *_bytes: strides of the rings; *_tx: bytes one load delivers
    DwtSource dw;
    EpiConfig e2;
    int K;                                     // hidden channels (the pointwise reduction length)
    const int8_t *res;
    int8_t *out;
    long long ops, rps;                        // output / residual pixel strides in bytes
};

// Byte offset of 16-byte chunk `chunk` of row `m` in a K-major operand whose rows are `pitch` bytes (= the swizzle width).
__device__ __forceinline__ uint32_t swz_off(int m, int chunk, int pitch)
{
    const int x = pitch == 128 ? (m & 7) : (pitch == 64 ? ((m >> 1) & 3) : ((m >> 2) & 1));
    return (uint32_t)(m * pitch + ((chunk ^ x) << 4));
}

template <int S, int CBT>
__global__ void __launch_bounds__(DP_THREADS, 1)
dwpw_kernel(const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_w2, const __grid_constant__ DpParams p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t *a0 = smem;                                              // two A operands of a_bytes (1024-aligned)
    uint8_t *w20 = a0 + 2 * (size_t)p.a_bytes;                       // two filter blocks of w2_bytes (1024-aligned)
    uint8_t *patch0 = w20 + DP_STAGES * (size_t)p.w2_bytes;          // two input patches
    uint8_t *aux = patch0 + DP_STAGES * (size_t)p.patch_bytes;
    FastParam *fast_s = (FastParam *)aux;                            // n_pad entries
    uint64_t *bars = (uint64_t *)(aux + sizeof(FastParam) * (size_t)p.n_pad);
    uint64_t *pfull = bars, *pempty = bars + 2, *wfull = bars + 4, *wempty = bars + 6, *afull = bars + 8, *aempty = bars + 10;
    uint64_t *dfull = bars + 12, *dempty = bars + 13;
    uint32_t *tmem_slot = (uint32_t *)(bars + 14);
    int *slow_flag = (int *)(tmem_slot + 1);
    volatile int *abort_flag = (volatile int *)(slow_flag + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int CB = CBT ? CBT : p.CB;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; s++) {
            mbar_init(smem_u32(&pfull[s]), 1);
            mbar_init(smem_u32(&pempty[s]), DP_DW_WARPS);
            mbar_init(smem_u32(&wfull[s]), 1);
            mbar_init(smem_u32(&wempty[s]), 1);
            mbar_init(smem_u32(&afull[s]), DP_DW_WARPS);
            mbar_init(smem_u32(&aempty[s]), 1);
        }
        mbar_init(smem_u32(dfull), 1);
        mbar_init(smem_u32(dempty), 4);
        *slow_flag = 0;
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1)
        tmem_alloc(smem_u32(tmem_slot), p.tmem_cols);
    __syncthreads(); // the flags are zero before anybody raises one
    // the A operands start as zeros: the depthwise warps write CB bytes of every row, the columns between CB and the
    // row pitch stay zero for the whole launch, so whatever the filter block holds there contributes nothing
    for (int i = threadIdx.x; i < 2 * p.a_bytes / 16; i += DP_THREADS) ((uint4 *)a0)[i] = make_uint4(0u, 0u, 0u, 0u);
    stage_fast_params(p.e2, fast_s, p.cout, p.n_pad, (int)threadIdx.x, DP_THREADS, slow_flag);
    fence_async_smem();
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const bool fast2 = !*slow_flag && !p.e2.half_even && p.K <= 32768;

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            uint32_t phase = 0;
            int stage = 0, cb = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
                const int xt = t % p.xtiles, r = t / p.xtiles;
                const int yt = r % p.ytiles, nblk = r / p.ytiles;
                for (cb = 0; cb < p.cblocks; cb++) {
                    if (!mbar_wait(smem_u32(&pempty[stage]), phase ^ 1) || !mbar_wait(smem_u32(&wempty[stage]), phase ^ 1)) {
                        ok = false;
                        break;
                    }
                    const uint32_t pb = smem_u32(&pfull[stage]), wb = smem_u32(&wfull[stage]);
                    mbar_arrive_expect_tx(pb, (uint32_t)p.patch_tx);
                    tma_load_4d(smem_u32(patch0 + (size_t)stage * p.patch_bytes), &map_in, cb * CB, xt * p.TW * S - p.pl, yt * p.TH * S - p.pt, nblk * p.NB, pb);
                    mbar_arrive_expect_tx(wb, (uint32_t)p.w2_tx);
                    tma_load_2d(smem_u32(w20 + (size_t)stage * p.w2_bytes), &map_w2, cb * CB, 0, wb);
                    if (++stage == DP_STAGES)
                        stage = 0, phase ^= 1;
                }
            }
            if (!ok) {
                *abort_flag = 1;
                atomicExch(&g_dwpw_error, ESPDL_ERR_TIMEOUT);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t phase = 0, dphase = 0;
            int stage = 0;
            bool ok = true;
            const uint32_t idesc = idesc_i8(1, 1, 128, p.n_pad);
            for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
                // the accumulators of the previous tile have been read
                if (!mbar_wait(smem_u32(dempty), dphase ^ 1)) {
                    ok = false;
                    break;
                }
                fence_after();
                for (int cb = 0; cb < p.cblocks && ok; cb++) {
                    if (!mbar_wait(smem_u32(&afull[stage]), phase) || !mbar_wait(smem_u32(&wfull[stage]), phase)) {
                        ok = false;
                        break;
                    }
                    fence_after();
                    const uint32_t ab = smem_u32(a0 + (size_t)stage * p.a_bytes), wb = smem_u32(w20 + (size_t)stage * p.w2_bytes);
                    const uint64_t db = smem_desc_swizzled(wb, p.pitch);
                    for (int mb = 0; mb < p.MB; mb++) {
                        const uint64_t da = smem_desc_swizzled(ab + (uint32_t)(mb * 128 * p.pitch), p.pitch);
                        for (int k = 0; k < p.ksteps; k++)
                            mma_i8(tmem_base + (uint32_t)(mb * p.n_pad), da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (cb | k) != 0);
                    }
                    commit(smem_u32(&aempty[stage]));
                    commit(smem_u32(&wempty[stage]));
                    if (++stage == DP_STAGES)
                        stage = 0, phase ^= 1;
                }
                if (!ok)
                    break;
                commit(smem_u32(dfull));
                dphase ^= 1;
            }
            if (!ok) {
                *abort_flag = 1;
                atomicExch(&g_dwpw_error, ESPDL_ERR_TIMEOUT);
            }
        }
        __syncwarp();
    } else if (warp < DP_FIRST_DW_WARP) {
        // ------------------------------------------------------------ epilogue (warps 2..5, TMEM lanes 32 * (warp & 3) ...)
        const int lane_group = warp & 3;
        const int row = lane_group * 32 + lane;
        uint32_t dphase = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
            const int xt = t % p.xtiles, r = t / p.xtiles;
            const int yt = r % p.ytiles, nblk = r / p.ytiles;
            if (!mbar_wait(smem_u32(dfull), dphase)) {
                ok = false;
                break;
            }
            dphase ^= 1;
            fence_after();
            for (int mb = 0; mb < p.MB; mb++) {
                // pixel of this accumulator row
                const int m = mb * 128 + row;
                const int x = m % p.TW, rr = m / p.TW;
                const int y = rr % p.TH, nb = rr / p.TH;
                const int gx = xt * p.TW + x, gy = yt * p.TH + y, gn = nblk * p.NB + nb;
                const bool row_ok = m < p.m_valid && gx < p.OW && gy < p.OH && gn < p.N;
                const long long pix = ((long long)gn * p.OH + gy) * p.OW + gx;
                int8_t *orow = p.out + pix * p.ops;
                const int8_t *rrow = p.res ? p.res + pix * p.rps : nullptr;
                const uint32_t t0 = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(mb * p.n_pad);
                for (int c0 = 0; c0 < p.n_pad; c0 += 16) {
                    int32_t v[16];
                    ld16(t0 + c0, v);
                    ld_wait16(v);
                    uint32_t pk[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                    if (fast2) {
                        if (p.e2.relu)
                            requant16_fast<true>(v, fast_s + c0, pk);
                        else
                            requant16_fast<false>(v, fast_s + c0, pk);
                    } else {
                        requant16_general(v, p.e2, c0, p.cout, pk);
                    }
                    const int count = min(16, p.cout - c0);
                    if (row_ok && count > 0) {
                        if (rrow) { // folded Add: saturating byte sums with the residual's row
#pragma unroll
                            for (int j = 0; j < 16; j++)
                                if (j < count) {
                                    const int sum = (int)(int8_t)(pk[j >> 2] >> (8 * (j & 3))) + (int)rrow[c0 + j];
                                    pk[j >> 2] = (pk[j >> 2] & ~(0xffu << (8 * (j & 3)))) | (((uint32_t)max(-128, min(127, sum)) & 0xffu) << (8 * (j & 3)));
                                }
                        }
                        const uintptr_t amix = (uintptr_t)(orow + c0) | 16u;
                        store_bytes(orow + c0, pk, count, (int)(amix & (~amix + 1)));
                    }
                }
            }
            fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(smem_u32(dempty));
        }
        if (!ok && lane == 0) {
            *abort_flag = 1;
            atomicExch(&g_dwpw_error, ESPDL_ERR_TIMEOUT);
        }
    } else {
        // ------------------------------------------------------------ depthwise warps
        constexpr int RB = S == 1 ? 4 : 2; // output rows per band
        const int tid = threadIdx.x - DP_FIRST_DW_WARP * 32;
        const int W4 = CB >> 2;
        const bool active = tid < p.items;
        const int cw = tid % W4;
        int r = tid / W4;
        const int seg = r % p.nseg;
        r /= p.nseg;
        const int band = r % p.nbands, nb = r / p.nbands;
        const int in_row_words = p.IW * W4;
        const int in_off = ((nb * p.IH + band * RB * S) * p.IW + seg * p.L * S) * W4 + cw; // words from the patch
        const int m0 = (nb * p.TH + band * RB) * p.TW + seg * p.L;                           // A row of (band row 0, run column 0)
        const int chunk = cw >> 2;
        const uint32_t within = (uint32_t)((cw & 3) << 2);
        const int floor_q = p.dw.relu ? 0 : INT_MIN;
        const int pitch = p.pitch, TW = p.TW;
        uint32_t phase = 0;
        int stage = 0;
        bool dead = false; // a wait expired: keep the barriers matched, touch nothing
        DwtConsts<S> k;
        for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x) {
            for (int cb = 0; cb < p.cblocks; cb++) {
                if (active && !dead)
                    dwt_load_consts<S>(k, p.dw, cb * CB + cw * 4);
                if (!dead && (!mbar_wait(smem_u32(&pfull[stage]), phase) || !mbar_wait(smem_u32(&aempty[stage]), phase ^ 1))) {
                    dead = true;
                    *abort_flag = 1;
                    if (lane == 0)
                        atomicExch(&g_dwpw_error, ESPDL_ERR_TIMEOUT);
                }
                if (!dead && *abort_flag)
                    dead = true;
                if (active && !dead) {
                    const uint32_t *patch = (const uint32_t *)(patch0 + (size_t)stage * p.patch_bytes);
                    uint8_t *abuf = a0 + (size_t)stage * p.a_bytes;
                    if (k.fast) {
                        auto store = [=](int ro, int x, uint32_t word) {
                            const int m = m0 + ro * TW + x;
                            *(uint32_t *)(abuf + swz_off(m, chunk, pitch) + within) = word;
                        };
                        dwt_walk<S, CBT / 4>(k, patch + in_off, store, in_row_words, W4, p.L, floor_q);
                    } else {
                        // channels outside the one-add-one-shift form: plain loops with the general requantisation
                        const int8_t *ip = (const int8_t *)(patch + in_off);
                        for (int ro = 0; ro < RB; ro++)
                            for (int x = 0; x < p.L; x++) {
                                uint32_t word = 0;
                                for (int i = 0; i < 4; i++) {
                                    const int c = cb * CB + cw * 4 + i;
                                    int32_t acc = 0;
                                    for (int ky = 0; ky < 3; ky++)
                                        for (int kx = 0; kx < 3; kx++)
                                            acc += (int)ip[((ro * S + ky) * p.IW + (x * S + kx)) * CB + i] * (int)p.dw.w[(ky * 3 + kx) * p.dw.C + c];
                                    const int e = p.dw.per_channel ? p.dw.ew[c] : p.dw.ew_scalar;
                                    const int shift = max(-31, min(31, p.dw.e_shift_base - e));
                                    const int32_t v = requant8(acc, p.dw.bias ? p.dw.bias[c] : 0, shift, p.dw.relu, p.dw.half_even);
                                    word |= ((uint32_t)v & 0xffu) << (8 * i);
                                }
                                const int m = m0 + ro * TW + x;
                                *(uint32_t *)(abuf + swz_off(m, chunk, pitch) + within) = word;
                            }
                    }
                }
                fence_async_smem(); // the operand words are visible to the tensor cores
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(smem_u32(&pempty[stage]));
                    mbar_arrive(smem_u32(&afull[stage]));
                }
                if (++stage == DP_STAGES)
                    stage = 0, phase ^= 1;
            }
        }
    }

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

EncodeTiledFn dp_encode()
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

size_t dp_smem_bytes(const DpParams &p)
{
    return 1024 + 2 * (size_t)p.a_bytes + DP_STAGES * ((size_t)p.w2_bytes + p.patch_bytes) + sizeof(FastParam) * (size_t)p.n_pad + 16 * 8 + 64;
}

// Tile shape: channel block CB (a divisor of the hidden channels, a multiple of 16, at most 128: one swizzled row of
// the A operand), NB images x TH x TW output pixels filling MB blocks of 128 accumulator rows, bands and runs such that
// the twelve depthwise warps each get one run.
bool dp_plan(const espdl_block_desc &d, DpParams &p)
{
    static std::mutex mu;
    static std::map<std::tuple<int, int, int, int, int, int>, DpParams> memo;
    const auto key = std::make_tuple(d.hidden_c, d.out_h, d.out_w, d.n, d.stride, d.out_c);
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = memo.find(key);
        if (it != memo.end()) {
            p = it->second;
            return p.items > 0;
        }
    }
    const int S = d.stride, RB = S == 1 ? 4 : 2, C = d.hidden_c;
    const int n_pad = (d.out_c + 15) / 16 * 16;
    DpParams best{};
    double best_score = -1.0;
    for (int CB = 16; CB <= 128 && CB <= C; CB += 16) {
        if (C % CB)
            continue;
        const int W4 = CB / 4;
        const int pitch = CB > 64 ? 128 : (CB > 32 ? 64 : 32);
        for (int MB = 1; MB <= 4; MB++) {
            if (MB * n_pad > 512)
                break;
            for (int NB = 1; NB <= 8 && NB <= d.n; NB++)
                for (int nbands = 1; nbands <= 8; nbands++) {
                    const int TH = nbands * RB;
                    if (TH > d.out_h + RB - 1)
                        break;
                    for (int nseg = 1; nseg <= 32; nseg++) {
                        const int threads = W4 * NB * nbands * nseg;
                        if (threads > DP_DW_THREADS)
                            break;
                        for (int L = 2; L <= 16; L++) {
                            const int TW = nseg * L;
                            if (TW > d.out_w + L - 1)
                                break;
                            const int m_valid = NB * TH * TW;
                            if (m_valid > MB * 128)
                                break;
                            if (m_valid <= (MB - 1) * 128)
                                continue; // a smaller MB covers it
                            const int IH = (TH - 1) * S + 3, IW = (TW - 1) * S + 3;
                            if (IW > 256 || IH > 256)
                                break;
                            DpParams q{};
                            q.patch_tx = NB * IH * IW * CB;
                            q.patch_bytes = (q.patch_tx + 127) & ~127;
                            q.w2_tx = n_pad * pitch;
                            q.w2_bytes = (q.w2_tx + 1023) & ~1023;
                            q.a_bytes = MB * 128 * pitch;
                            q.n_pad = n_pad;
                            if (dp_smem_bytes(q) > DP_SMEM_BUDGET)
                                break;
                            const int xt = (d.out_w + TW - 1) / TW, yt = (d.out_h + TH - 1) / TH, nbk = (d.n + NB - 1) / NB;
                            const double useful = ((double)d.out_w / (xt * TW)) * ((double)d.out_h / (yt * TH)) * ((double)d.n / (nbk * NB));
                            const double cols = S == 1 ? (L + 2.0) / L : (2.0 * L + 1.0) / (2.0 * L);
                            const double halo = ((double)IH * IW) / ((double)TH * S * TW * S);
                            const long long tiles = (long long)xt * yt * nbk;
                            const double waves = (double)tiles / num_sms();
                            const double tail = waves / ceil(waves);
                            const double rows = (double)m_valid / (MB * 128);
                            // a run costs its columns plus a fixed share per step (constants, barriers): longer runs amortise it
                            const double fixed = (double)L / (L + 1.5);
                            const double score = useful * ((double)threads / DP_DW_THREADS) / (0.6 + 0.4 * cols) / (0.75 + 0.25 * halo) * tail * (0.7 + 0.3 * rows) * fixed *
                                (CB >= 64 ? 1.0 : 0.85);
                            if (score > best_score + 1e-12) {
                                best_score = score;
                                q.S = S, q.CB = CB, q.pitch = pitch, q.ksteps = (CB + 31) / 32;
                                q.NB = NB, q.TH = TH, q.TW = TW, q.IH = IH, q.IW = IW, q.L = L, q.nseg = nseg, q.nbands = nbands, q.items = threads;
                                q.MB = MB, q.m_valid = m_valid;
                                q.cblocks = C / CB, q.nblocks = nbk, q.ytiles = yt, q.xtiles = xt;
                                q.total_tiles = tiles > 0x7fffffffll / 64 ? 0 : (int)tiles;
                                int cols_pow2 = 32;
                                while (cols_pow2 < MB * n_pad) cols_pow2 *= 2;
                                q.tmem_cols = cols_pow2;
                                best = q;
                            }
                        }
                    }
                }
        }
    }
    if (best_score < 0 || best.total_tiles == 0)
        best.items = 0;
    {
        std::lock_guard<std::mutex> lock(mu);
        memo[key] = best;
    }
    p = best;
    return p.items > 0;
}

template <int S, int CBT>
int dp_launch(const CUtensorMap &mi, const CUtensorMap &mw, const DpParams &p, size_t smem, int grid, cudaStream_t s)
{
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] { attr_err = cudaFuncSetAttribute(dwpw_kernel<S, CBT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(DP_SMEM_BUDGET + 2048)); });
    if (attr_err != cudaSuccess)
        return set_cuda_error(attr_err, "cudaFuncSetAttribute(dwpw_kernel)");
    if (smem < 120 * 1024)
        smem = 120 * 1024; // one CTA per SM, so that TMEM allocation never waits on a neighbour
    dwpw_kernel<S, CBT><<<grid, DP_THREADS, smem, s>>>(mi, mw, p);
    count_launch();
    return check_launch("dwpw");
}

template <int S>
int dp_dispatch(const CUtensorMap &mi, const CUtensorMap &mw, const DpParams &p, size_t smem, int grid, cudaStream_t s)
{
    switch (p.CB) {
    case 32: return dp_launch<S, 32>(mi, mw, p, smem, grid, s);
    case 48: return dp_launch<S, 48>(mi, mw, p, smem, grid, s);
    case 64: return dp_launch<S, 64>(mi, mw, p, smem, grid, s);
    case 96: return dp_launch<S, 96>(mi, mw, p, smem, grid, s);
    case 128: return dp_launch<S, 128>(mi, mw, p, smem, grid, s);
    default: return dp_launch<S, 0>(mi, mw, p, smem, grid, s);
    }
}

} // namespace

// The pair the kernel takes: no expand conv, int8, 3x3 depthwise of stride 1 or 2, hidden channels a multiple of 16,
// at most 256 output channels, round half up, no upper clamp below 127.
bool fused_dwpw_supported(const espdl_block_desc &d, bool has_expand)
{
    if (has_expand || d.dtype != ESPDL_DTYPE_INT8 || (d.stride != 1 && d.stride != 2) || d.hidden_c % 16 || d.hidden_c != d.in_c)
        return false;
    if (d.out_c < 1 || d.out_c > 256 || d.hidden_c > 32768 || d.pad_top < 0 || d.pad_left < 0 || d.pad_top > 255 || d.pad_left > 255)
        return false;
    if (d.round_mode != ESPDL_ROUND_HALF_UP || (d.dw_clip_max != 0 && d.dw_clip_max < 127) || getenv("ESPDL_B200_NO_DWPW"))
        return false;
    DpParams p;
    return dp_plan(d, p);
}

int fused_dwpw(const espdl_block_desc &d, cudaStream_t s)
{
    DpParams p;
    if (!dp_plan(d, p))
        return ESPDL_ERR_UNSUPPORTED;
    if (((uintptr_t)d.input % 16) || ((uintptr_t)d.project_filter % 16) || ((uintptr_t)d.dw_filter % 4))
        return ESPDL_ERR_UNSUPPORTED;
    if ((((d.per_channel >> 1) & 1) && !d.dw_filter_exponents) || (((d.per_channel >> 2) & 1) && !d.project_filter_exponents))
        return set_error_text(ESPDL_ERR_INVALID_ARG, "fused block: per-channel exponents requested without an exponent array");
    EncodeTiledFn enc = dp_encode();
    if (!enc)
        return set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point not found");
    p.N = d.n, p.OH = d.out_h, p.OW = d.out_w, p.cout = d.out_c, p.K = d.hidden_c;
    p.pt = d.pad_top, p.pl = d.pad_left;
    p.dw.C = d.hidden_c, p.dw.w = (const int8_t *)d.dw_filter, p.dw.bias = (const int32_t *)d.dw_bias, p.dw.ew = d.dw_filter_exponents, p.dw.lut = nullptr, p.dw.lut_stride = 0;
    p.dw.e_shift_base = d.dw_exponent - d.in_exponent, p.dw.ew_scalar = d.dw_filter_exponent, p.dw.per_channel = (d.per_channel >> 1) & 1;
    p.dw.relu = d.dw_activation == ESPDL_ACT_RELU, p.dw.half_even = 0;
    p.e2 = EpiConfig{d.project_bias, d.project_filter_exponents, nullptr, d.out_exponent - d.dw_exponent, d.project_filter_exponent, (d.per_channel >> 2) & 1,
                     d.project_activation == ESPDL_ACT_RELU, 0};
    p.res = (const int8_t *)d.residual, p.out = (int8_t *)d.output;
    p.ops = d.out_c, p.rps = d.out_c;
    CUtensorMap mi, mw;
    {
        cuuint64_t dims[4] = {(cuuint64_t)d.in_c, (cuuint64_t)d.in_w, (cuuint64_t)d.in_h, (cuuint64_t)d.n};
        cuuint64_t strides[3] = {(cuuint64_t)d.in_c, (cuuint64_t)d.in_c * d.in_w, (cuuint64_t)d.in_c * d.in_w * d.in_h};
        cuuint32_t box[4] = {(cuuint32_t)p.CB, (cuuint32_t)p.IW, (cuuint32_t)p.IH, (cuuint32_t)p.NB};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        if (enc(&mi, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(d.input), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(fused block input)");
    }
    {
        // the pointwise filter [out_c][hidden_c]: a box of `pitch` channels x n_pad rows; rows past out_c and channels past
        // hidden_c come back as zeros
        cuuint64_t dims[2] = {(cuuint64_t)d.hidden_c, (cuuint64_t)d.out_c};
        cuuint64_t strides[1] = {(cuuint64_t)d.hidden_c};
        cuuint32_t box[2] = {(cuuint32_t)p.pitch, (cuuint32_t)p.n_pad};
        cuuint32_t estr[2] = {1, 1};
        const CUtensorMapSwizzle sw = p.pitch == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (p.pitch == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
        if (enc(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(d.project_filter), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(fused block pointwise filter)");
    }
    const size_t smem = dp_smem_bytes(p);
    const int grid = min(p.total_tiles, num_sms());
    return d.stride == 1 ? dp_dispatch<1>(mi, mw, p, smem, grid, s) : dp_dispatch<2>(mi, mw, p, smem, grid, s);
}

} // namespace espdl
