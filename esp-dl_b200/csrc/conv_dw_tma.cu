// 3x3 DepthwiseConv2D, int8, stride 1 or 2, fed by TMA: the default depthwise kernel for NHWC tensors whose channel
// count is a multiple of 16.
// Replaces dl::base::depthwise_conv2d<int8_t,...> (esp-dl/dl/base/dl_base_depthwise_conv2d.cpp:47-66, shell
// esp-dl/dl/base/dl_base.hpp:1209-2107): out[y,x,c] = sat8(act(rnd((sum_{ky,kx} in[y*s+ky-pt, x*s+kx-pl, c] * w[ky,kx,c] + bias[c]) >> shift[c]))),
// taps outside the image contribute nothing.
//
// The op moves two bytes per output and needs nine MACs for them: it is bound by HBM if and only if the arithmetic keeps
// up.  dw3x3_dp4a_kernel (conv_dw.cu) reads its columns straight from global memory and stalls on those loads with 16
// warps per SM; here one persistent CTA per SM splits the roles:
//   warp 16     producer: one 4-D TMA box per tile brings the input patch (NB images x IH rows x IW columns x CB
//               channels, zero-filled outside the image, so padding needs no code) into a two-stage shared-memory
//               ring - a whole tile of loads is in flight while the previous one is being computed;
//   warps 0-15  consumers: a thread owns four channels (one 32-bit word of a pixel), a band of output rows and a run
//               of L output columns of the tile, fixed for the whole launch.  It walks along its run exactly as
//               dw3x3_dp4a_kernel does (byte-transposed columns, dp4a against the filter columns, accumulators that
//               start from bias + 2^(shift-1)), reading shared memory with immediate offsets and writing the
//               requantised words into an output tile in shared memory, which one TMA store per tile moves to global
//               memory (clipped at the image border, so ragged tiles need no code either).
// Every mbarrier wait is bounded; a wait that expires records ESPDL_ERR_TIMEOUT, raises a CTA-wide flag that every role
// reads at a point all of them pass, and the CTA leaves with its barriers matched.
#include "dw_walk.cuh"
#include "tc_common.cuh"

#include <cmath>
#include <map>
#include <mutex>
#include <tuple>

namespace espdl {

__device__ int g_dwt_error = 0;

int read_and_clear_device_error_dw()
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_dwt_error, sizeof(int)) != cudaSuccess)
        return 0;
    if (v) {
        int zero = 0;
        cudaMemcpyToSymbol(g_dwt_error, &zero, sizeof(int));
    }
    return v;
}

namespace {

using namespace tc;
using namespace dwt;

constexpr int DWT_CONSUMER_WARPS = 16;
constexpr int DWT_CONSUMERS = DWT_CONSUMER_WARPS * 32;
constexpr int DWT_THREADS = DWT_CONSUMERS + 32;
constexpr int DWT_STAGES = 2;
constexpr int DWT_RING = 8; // tile numbers on their way from the producer to the consumers (more than DWT_STAGES)
constexpr size_t DWT_SMEM_BUDGET = 200 * 1024;

struct DwtParams {
    int S, CB, NB, TH, TW, IH, IW, L, nseg, nbands, items;
    int cblocks, nblocks, ytiles, xtiles, tiles_per_cb, total_tiles;
    int pt, pl;
    int stage_bytes, out_bytes, tx_bytes; // patch stride in the ring, output tile size, bytes one patch load delivers
    long long wait_limit;                 // cycles a wait may take (WAIT_LIMIT_CYCLES; shorter only in the expiry test)
    int withhold_arrive;                  // expiry test: consumer warp 0 never reports a patch as read, so the producer's wait runs out
    unsigned *sched;                      // {next tile, CTAs done}: the tiles from static_tiles on are handed out by this counter; null = fixed walk
    int static_tiles;                     // tiles walked in the fixed order (a multiple of the grid size)
    DwtSource src;
};

__device__ __forceinline__ void tma_store_4d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2, int c3)
{
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map), "r"(src), "r"(c0), "r"(c1),
                 "r"(c2), "r"(c3)
                 : "memory");
}

// The same run for channels outside the one-add-one-shift form (a shift outside 1..24, a huge bias, half-even rounding
// or a fused table): plain loops over the patch with the general requantisation.
__device__ __noinline__ void dwt_walk_general(const DwtParams &pp, int S, const int8_t *ip, int8_t *op, int in_row_bytes, int out_row_bytes, int c0, int L)
{
    const DwtSource &p = pp.src;
    const int rows_out = S == 1 ? 4 : 2;
    for (int ro = 0; ro < rows_out; ro++)
        for (int x = 0; x < L; x++)
            for (int i = 0; i < 4; i++) {
                int32_t acc = 0;
                for (int ky = 0; ky < 3; ky++)
                    for (int kx = 0; kx < 3; kx++)
                        acc += (int)ip[(ro * S + ky) * in_row_bytes + (x * S + kx) * pp.CB + i] * (int)p.w[(ky * 3 + kx) * p.C + c0 + i];
                const int e = p.per_channel ? p.ew[c0 + i] : p.ew_scalar;
                const int shift = max(-31, min(31, p.e_shift_base - e));
                int32_t v = requant8(acc, p.bias ? p.bias[c0 + i] : 0, shift, p.relu, p.half_even);
                if (p.lut)
                    v = p.lut[(long long)(c0 + i) * p.lut_stride + ((uint8_t)v ^ 0x80u)];
                op[ro * out_row_bytes + x * pp.CB + i] = (int8_t)v;
            }
}

template <int S, int CBT>
__global__ void __launch_bounds__(DWT_THREADS, 1)
dw3x3_tma_kernel(const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_out, const __grid_constant__ DwtParams p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte aligned start, found by offset so that every pointer below is still known to be shared memory
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t *patch0 = smem;                                           // DWT_STAGES patches of stage_bytes
    uint8_t *out0 = patch0 + (size_t)DWT_STAGES * p.stage_bytes;      // two output tiles of out_bytes
    uint64_t *bars = (uint64_t *)(out0 + 2 * (size_t)p.out_bytes);
    uint64_t *full_bar = bars, *empty_bar = bars + DWT_STAGES;
    volatile int *abort_flag = (volatile int *)(bars + 2 * DWT_STAGES);
    volatile int *tile_ring = abort_flag + 1; // DWT_RING tile numbers, producer -> consumers (published by the "full" arrive)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < DWT_STAGES; s++) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), DWT_CONSUMER_WARPS);
        }
        *abort_flag = 0;
        for (int i = 0; i < DWT_RING; i++) tile_ring[i] = 0; // never negative before the producer says so
        fence_barrier_init();
    }
    if (threadIdx.x == 32) {
        prefetch_tensormap(&map_in);
        prefetch_tensormap(&map_out);
    }
    __syncthreads();
    const int CB = CBT ? CBT : p.CB;
    if (threadIdx.x == 0)
        grid_dep_launch(); // set up: the next kernel's CTAs may take SMs as they become free

    if (warp == DWT_CONSUMER_WARPS) {
        grid_dep_wait(); // the previous kernel's output (and its use of the tile counter) before the first load
        // ------------------------------------------------------------ producer: the warp walks the tiles, lane 0 issues
        // Tiles below p.static_tiles go round the CTAs in the fixed order; the rest is handed out by a global counter, one
        // number per tile and asked for one tile ahead, so that an SM that runs slower than the others ends with fewer tiles.
        int stage = 0, local = 0;
        uint32_t phase = 0;
        bool handed = false, ok = true;
        auto after = [&](int cur) {
            if (!handed && cur + (int)gridDim.x < p.static_tiles)
                return cur + (int)gridDim.x;
            if (!p.sched)
                return handed || cur + (int)gridDim.x >= p.total_tiles ? p.total_tiles : cur + (int)gridDim.x;
            handed = true;
            int v = 0;
            if (lane == 0)
                v = p.static_tiles + (int)atomicAdd(p.sched, 1u);
            return __shfl_sync(0xffffffffu, v, 0);
        };
        int t = blockIdx.x;
        int next = after(t);
        for (; t < p.total_tiles; local++) {
            if (*abort_flag) {
                ok = false;
                break;
            }
            if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, p.wait_limit)) {
                *abort_flag = 1;
                if (lane == 0)
                    atomicExch(&g_dwt_error, ESPDL_ERR_TIMEOUT);
                ok = false;
                break;
            }
            const int cb = t / p.tiles_per_cb, t_in_cb = t - cb * p.tiles_per_cb;
            const int xt = t_in_cb % p.xtiles, r = t_in_cb / p.xtiles;
            const int yt = r % p.ytiles, nblk = r / p.ytiles;
            if (lane == 0) {
                tile_ring[local & (DWT_RING - 1)] = t;
                const uint32_t bar = smem_u32(&full_bar[stage]);
                mbar_arrive_expect_tx(bar, (uint32_t)p.tx_bytes);
                tma_load_4d(smem_u32(patch0 + (size_t)stage * p.stage_bytes), &map_in, cb * CB, xt * p.TW * S - p.pl, yt * p.TH * S - p.pt, nblk * p.NB, bar);
            }
            if (++stage == DWT_STAGES)
                stage = 0, phase ^= 1;
            t = next;
            if (t < p.total_tiles)
                next = after(t);
        }
        // end of the walk: one stage without data whose ring entry is negative
        if (ok && mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, p.wait_limit)) {
            if (lane == 0) {
                tile_ring[local & (DWT_RING - 1)] = -1;
                mbar_arrive(smem_u32(&full_bar[stage]));
            }
        }
        __syncwarp();
        if (p.sched && lane == 0) {
            // the last CTA's producer leaves the counters as it found them (it is also the thread that asked for tiles)
            __threadfence();
            if (atomicAdd(p.sched + 1, 1u) == gridDim.x - 1) {
                p.sched[0] = 0;
                p.sched[1] = 0;
            }
        }
        __syncwarp();
        return;
    }

    // ---------------------------------------------------------------- consumers
    constexpr int RB = S == 1 ? 4 : 2; // output rows per band
    const int tid = threadIdx.x;
    const int W4 = CB >> 2;
    const bool active = tid < p.items;
    const int cw = tid % W4;
    int r = tid / W4;
    const int seg = r % p.nseg;
    r /= p.nseg;
    const int band = r % p.nbands, nb = r / p.nbands;
    const int in_row_words = p.IW * W4, out_row_words = p.TW * W4;
    const int in_off = ((nb * p.IH + band * RB * S) * p.IW + seg * p.L * S) * W4 + cw;   // words from the patch
    const int out_off = ((nb * p.TH + band * RB) * p.TW + seg * p.L) * W4 + cw;          // words from the output tile
    const int floor_q = p.src.relu ? 0 : INT_MIN;

    DwtConsts<S> k;
    int have_cb = -1;
    int stage = 0;
    uint32_t phase = 0;
    for (int local = 0;; local++) {
        if (!mbar_wait(smem_u32(&full_bar[stage]), phase, p.wait_limit)) {
            // the patch never came: note it and leave at the barrier below, where all threads see the flag together
            *abort_flag = 1;
            if (lane == 0)
                atomicExch(&g_dwt_error, ESPDL_ERR_TIMEOUT);
        }
        const int t = *abort_flag ? 0 : tile_ring[local & (DWT_RING - 1)];
        if (t < 0)
            break;
        const int cb = t / p.tiles_per_cb, t_in_cb = t - cb * p.tiles_per_cb;
        if (cb != have_cb && active) {
            dwt_load_consts<S>(k, p.src, cb * CB + cw * 4);
            have_cb = cb;
        }
        const uint32_t *patch = (const uint32_t *)(patch0 + (size_t)stage * p.stage_bytes);
        uint32_t *obuf = (uint32_t *)(out0 + (size_t)(local & 1) * p.out_bytes);
        if (active) {
            if (k.fast) {
                uint32_t *op = obuf + out_off;
                const int cb4 = CBT ? CBT / 4 : W4;
                auto store = [=](int ro, int x, uint32_t word) { op[ro * out_row_words + x * cb4] = word; };
                dwt_walk<S, CBT / 4>(k, patch + in_off, store, in_row_words, W4, p.L, floor_q);
            }
            else
                dwt_walk_general(p, S, (const int8_t *)(patch + in_off), (int8_t *)(obuf + out_off), in_row_words * 4, out_row_words * 4,
                                 cb * CB + cw * 4, p.L);
        }
        __syncwarp();
        if (lane == 0 && !(p.withhold_arrive && warp == 0))
            mbar_arrive(smem_u32(&empty_bar[stage])); // this warp has read the patch
        fence_async_smem();                           // the output words are visible to the TMA unit
        if (tid == 0)
            bulk_wait_read_all(); // the previous tile's store has left its buffer, which the next tile writes
        named_bar(1, DWT_CONSUMERS);
        if (*abort_flag)
            break;
        if (tid == 0) {
            const int xt = t_in_cb % p.xtiles, rr = t_in_cb / p.xtiles;
            tma_store_4d(&map_out, smem_u32(obuf), cb * CB, xt * p.TW, (rr % p.ytiles) * p.TH, (rr / p.ytiles) * p.NB);
            bulk_commit();
        }
        if (++stage == DWT_STAGES)
            stage = 0, phase ^= 1;
    }
    if (tid == 0)
        bulk_wait_all(); // shared memory stays allocated until the last store has left it
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn dwt_encode()
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

size_t dwt_smem_bytes(const DwtParams &p) { return 1024 + (size_t)DWT_STAGES * p.stage_bytes + 2 * (size_t)p.out_bytes + 2 * DWT_STAGES * 8 + 64 + DWT_RING * 4; }

// Tile shape: channel block CB, NB images, nbands bands of rows, nseg runs of L columns - the combination that keeps the
// most consumer threads at useful work (one run per thread) within the shared-memory budget.
bool dwt_plan(const espdl_conv_desc &d, DwtParams &p)
{
    static std::mutex mu;
    static std::map<std::tuple<int, int, int, int, int>, DwtParams> memo;
    const auto key = std::make_tuple(d.in_c, d.out_h, d.out_w, d.n, d.stride_h);
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = memo.find(key);
        if (it != memo.end()) {
            p = it->second;
            return p.items > 0;
        }
    }
    const int S = d.stride_h, RB = S == 1 ? 4 : 2;
    const int C = d.in_c;
    DwtParams best{};
    double best_score = -1.0;
    for (int CB = 16; CB <= 256 && CB <= C; CB += 16) {
        if (C % CB)
            continue;
        const int W4 = CB / 4;
        for (int NB = 1; NB <= 8 && NB <= d.n; NB++)
            for (int nbands = 1; nbands <= 8; nbands++) {
                const int TH = nbands * RB;
                if (TH > d.out_h + RB - 1)
                    break;
                for (int nseg = 1; nseg <= 32; nseg++) {
                    const int threads = W4 * NB * nbands * nseg;
                    if (threads > DWT_CONSUMERS)
                        break;
                    for (int L = 2; L <= 32; L++) {
                        const int TW = nseg * L;
                        if (TW > d.out_w + L - 1)
                            break;
                        const int IH = (TH - 1) * S + 3, IW = (TW - 1) * S + 3;
                        if (IW > 256 || IH > 256 || TW > 256)
                            break;
                        DwtParams q{};
                        q.tx_bytes = NB * IH * IW * CB;
                        q.stage_bytes = (q.tx_bytes + 127) & ~127;
                        q.out_bytes = (NB * TH * TW * CB + 127) & ~127;
                        if (dwt_smem_bytes(q) > DWT_SMEM_BUDGET)
                            break;
                        const int xt = (d.out_w + TW - 1) / TW, yt = (d.out_h + TH - 1) / TH, nbk = (d.n + NB - 1) / NB;
                        const double useful = ((double)d.out_w / (xt * TW)) * ((double)d.out_h / (yt * TH)) * ((double)d.n / (nbk * NB));
                        const double cols = S == 1 ? (L + 2.0) / L : (2.0 * L + 1.0) / (2.0 * L); // columns transposed per column needed
                        const double halo = ((double)IH * IW) / ((double)TH * S * TW * S);           // bytes fetched per byte needed
                        const long long tiles = (long long)xt * yt * nbk * (C / CB);
                        const double waves = (double)tiles / num_sms();
                        const double tail = waves / ceil(waves);                                     // the last wave's fill
                        const double row_bytes = CB >= 64 ? 1.0 : 0.8;                               // narrow TMA rows move slower
                        const double score = useful * ((double)threads / DWT_CONSUMERS) / cols / (0.75 + 0.25 * halo) * tail * row_bytes;
                        if (score > best_score + 1e-12) {
                            best_score = score;
                            q.S = S, q.CB = CB, q.NB = NB, q.TH = TH, q.TW = TW, q.IH = IH, q.IW = IW, q.L = L, q.nseg = nseg, q.nbands = nbands;
                            q.items = threads;
                            q.cblocks = C / CB, q.nblocks = nbk, q.ytiles = yt, q.xtiles = xt;
                            q.tiles_per_cb = xt * yt * nbk;
                            q.total_tiles = tiles > 0x7fffffffll ? 0 : (int)tiles;
                            best = q;
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
int dwt_launch(const CUtensorMap &mi, const CUtensorMap &mo, const DwtParams &p, size_t smem, int grid, cudaStream_t s)
{
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] { attr_err = cudaFuncSetAttribute(dw3x3_tma_kernel<S, CBT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(DWT_SMEM_BUDGET + 2048)); });
    if (attr_err != cudaSuccess)
        return set_cuda_error(attr_err, "cudaFuncSetAttribute(dw3x3_tma_kernel)");
    launch_overlapped(dw3x3_tma_kernel<S, CBT>, dim3(grid), dim3(DWT_THREADS), smem, s, mi, mo, p);
    count_launch();
    return check_launch("dw3x3_tma");
}

template <int S>
int dwt_dispatch(const CUtensorMap &mi, const CUtensorMap &mo, const DwtParams &p, size_t smem, int grid, cudaStream_t s)
{
    switch (p.CB) {
    case 32: return dwt_launch<S, 32>(mi, mo, p, smem, grid, s);
    case 64: return dwt_launch<S, 64>(mi, mo, p, smem, grid, s);
    case 96: return dwt_launch<S, 96>(mi, mo, p, smem, grid, s);
    case 128: return dwt_launch<S, 128>(mi, mo, p, smem, grid, s);
    case 144: return dwt_launch<S, 144>(mi, mo, p, smem, grid, s);
    case 192: return dwt_launch<S, 192>(mi, mo, p, smem, grid, s);
    default: return dwt_launch<S, 0>(mi, mo, p, smem, grid, s);
    }
}

} // namespace

bool conv2d_dw_tma_supported(const espdl_conv_desc &d)
{
    if (d.dtype != ESPDL_DTYPE_INT8 || d.group == 1 || d.kh != 3 || d.kw != 3 || d.dilation_h != 1 || d.dilation_w != 1)
        return false;
    if (d.stride_h != d.stride_w || (d.stride_h != 1 && d.stride_h != 2))
        return false;
    const int ips = d.in_pixel_stride ? d.in_pixel_stride : d.in_c, ops = d.out_pixel_stride ? d.out_pixel_stride : d.out_c;
    if (d.in_c % 16 || ips % 16 || ops % 16 || ((uintptr_t)d.input % 16) || ((uintptr_t)d.output % 16) || ((uintptr_t)d.filter % 4))
        return false;
    if (d.pad_top > 255 || d.pad_left > 255 || getenv("ESPDL_B200_NO_DW_TMA"))
        return false;
    // The TMA unit moves 32-byte runs at a fraction of the speed of wider ones (112x112x32, stride 1: 424 us here against
    // 210 us for the kernel that reads global memory directly), so narrow tensors stay with that kernel.
    if (d.in_c < 64 && !getenv("ESPDL_B200_DW_TMA_NARROW"))
        return false;
    DwtParams p;
    return dwt_plan(d, p);
}

int conv2d_dw_tma(const espdl_conv_desc &d, cudaStream_t s)
{
    DwtParams p;
    if (!conv2d_dw_tma_supported(d) || !dwt_plan(d, p))
        return ESPDL_ERR_UNSUPPORTED;
    EncodeTiledFn enc = dwt_encode();
    if (!enc)
        return set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point not found");
    const int ips = d.in_pixel_stride ? d.in_pixel_stride : d.in_c, ops = d.out_pixel_stride ? d.out_pixel_stride : d.out_c;
    p.pt = d.pad_top, p.pl = d.pad_left;
    // ESPDL_B200_DEBUG_WAIT_EXPIRY=<milliseconds>: the test of the bounded waits.  One arrival is withheld and the limit is
    // that short, so the producer's wait runs out, the CTA raises its flag and every role leaves; espdl_b200_stream_sync
    // then reports ESPDL_ERR_TIMEOUT.  Nothing traps, nothing waits without a limit.
    const char *expiry = getenv("ESPDL_B200_DEBUG_WAIT_EXPIRY");
    p.withhold_arrive = expiry && atoi(expiry) > 0 ? 1 : 0;
    p.wait_limit = p.withhold_arrive ? (long long)atoi(expiry) * 2000000ll : WAIT_LIMIT_CYCLES;
    p.src.C = d.in_c;
    p.src.w = (const int8_t *)d.filter, p.src.bias = (const int32_t *)d.bias, p.src.ew = d.filter_exponents, p.src.lut = d.lut, p.src.lut_stride = d.lut_channel_stride;
    p.src.e_shift_base = d.out_exponent - d.in_exponent;
    p.src.ew_scalar = d.filter_exponent, p.src.per_channel = d.per_channel;
    p.src.relu = d.activation == ESPDL_ACT_RELU, p.src.half_even = d.round_mode == ESPDL_ROUND_HALF_EVEN;
    CUtensorMap mi, mo;
    {
        cuuint64_t dims[4] = {(cuuint64_t)d.in_c, (cuuint64_t)d.in_w, (cuuint64_t)d.in_h, (cuuint64_t)d.n};
        cuuint64_t strides[3] = {(cuuint64_t)ips, (cuuint64_t)ips * d.in_w, (cuuint64_t)ips * d.in_w * d.in_h};
        cuuint32_t box[4] = {(cuuint32_t)p.CB, (cuuint32_t)p.IW, (cuuint32_t)p.IH, (cuuint32_t)p.NB};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        if (enc(&mi, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(d.input), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(depthwise input)");
    }
    {
        cuuint64_t dims[4] = {(cuuint64_t)d.out_c, (cuuint64_t)d.out_w, (cuuint64_t)d.out_h, (cuuint64_t)d.n};
        cuuint64_t strides[3] = {(cuuint64_t)ops, (cuuint64_t)ops * d.out_w, (cuuint64_t)ops * d.out_w * d.out_h};
        cuuint32_t box[4] = {(cuuint32_t)p.CB, (cuuint32_t)p.TW, (cuuint32_t)p.TH, (cuuint32_t)p.NB};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        if (enc(&mo, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, d.output, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(depthwise output)");
    }
    const size_t smem = dwt_smem_bytes(p);
    const int grid = min(p.total_tiles, num_sms());
    // three quarters of the tiles in the fixed order, the last quarter to whichever SM is free
    p.sched = p.total_tiles >= 4 * grid ? sched_counters(s) : nullptr;
    p.static_tiles = p.sched ? (int)((long long)p.total_tiles * 3 / 4 / grid) * grid : p.total_tiles;
    return d.stride_h == 1 ? dwt_dispatch<1>(mi, mo, p, smem, grid, s) : dwt_dispatch<2>(mi, mo, p, smem, grid, s);
}

} // namespace espdl
