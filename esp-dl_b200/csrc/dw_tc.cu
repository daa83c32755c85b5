// 3x3 DepthwiseConv2D (stride 1 or 2, int8) on the tensor cores.
//
// On CUDA cores a depthwise 3x3 costs 9 multiply-adds plus unpacking per output byte, which caps the op far below
// HBM speed.  Here the nine taps run as tcgen05.mma kind::i8 instructions with a DIAGONAL B operand:
//
//     D[pixel, c] += sum_k A_tap[pixel, k] * diag(w_tap)[k, c]        (32 channels per instruction, K = N = 32)
//
// 31/32 of the multiplies are by zero, but the tensor pipe has two orders of magnitude more int8 throughput than the
// op needs, and the CUDA cores are left with just the requantising epilogue (one add, one shift, a pack per output).
//
// Data movement: a work unit is a tile of 128 output pixels (R rows x P columns of a P-pitch grid, P = 16 or 32, of
// which the last columns are overhang) x a group of WC = 32, 64 or 128 channels.  ONE 4-D TMA box brings the input
// window of the whole channel group into shared memory as a plane of consecutive WC-byte pixels with the WC-byte
// swizzle - the K-major swizzled operand layout whose rows are pixels - so a filter tap (ky, kx) is the SAME plane
// with the descriptor's start address moved by (ky*P + kx) rows, and a 32-channel block is a 32-byte step inside
// the row.  (Rows of full 128 bytes matter: the TMA unit moves 16- or 32-byte rows at a fraction of HBM speed.)
// Image borders cost nothing: coordinates outside the tensor are zero-filled by the
// TMA unit, which is ESP-DL's "skip taps outside the image" rule (esp-dl/dl/base/dl_base.hpp:1209-2107).
// Stride 2 loads four parity planes (TMA element strides of 2), so that consecutive OUTPUT pixels are again
// consecutive rows.
//
// Replaces dl::base::depthwise_conv2d<int8_t,...> (esp-dl/dl/base/dl_base_depthwise_conv2d.cpp:9-66,760-881) for
// these shapes; roles, barriers, bounded waits and the epilogue are those of the pointwise tile kernel (gemm_tc.cu).
#include "tc_common.cuh"

#include <mutex>

namespace espdl {

__device__ int g_dw_tc_error = 0;

int read_and_clear_device_error_dw()
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_dw_tc_error, sizeof(int)) != cudaSuccess)
        return 0;
    if (v) {
        int zero = 0;
        cudaMemcpyToSymbol(g_dw_tc_error, &zero, sizeof(int));
    }
    return v;
}

namespace {

using namespace tc;

constexpr int DW_THREADS = 64 + 16 * 32;
constexpr int DW_CG = 128;      // TMEM columns per accumulator buffer = most channels a work unit can hold
constexpr int DW_ACC = 4;       // accumulator buffers (4 x 128 columns = all of TMEM)
constexpr int DW_MAX_STAGES = 8;

struct DwTcParams {
    int n, ih, iw, c, oh, ow;
    int S, P, R;            // stride, grid pitch (columns per tile row incl. overhang), output rows per tile
    int two;                // valid output columns per tile row
    int rows_in;            // plane rows loaded per tile
    int plane_px;           // pixels reserved per plane in shared memory (incl. one slack row)
    int phases;             // S*S parity planes per channel chunk
    int xtiles, ytiles, ncg;
    int cg;                 // channels per work unit = bytes per plane row = swizzle width: 32, 64 or 128
    int stages;
    int pt, pl;
    long long ops;
    void *out;
    const int8_t *w;        // [3][3][C]
    EpiConfig epi;
};

__global__ void __launch_bounds__(DW_THREADS, 1) dw_tc_kernel(const __grid_constant__ CUtensorMap map_in, const DwTcParams p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int plane_bytes = p.plane_px * p.cg;
    const int stage_bytes = p.phases * plane_bytes;
    uint8_t *b_smem = smem + (size_t)p.stages * stage_bytes;             // [cblock 4][tap 9][1024]
    FastParam *fast_s = (FastParam *)(b_smem + 4 * 9 * 1024);            // DW_CG entries
    uint64_t *bars = (uint64_t *)(fast_s + DW_CG);
    uint64_t *full_bar = bars, *empty_bar = bars + DW_MAX_STAGES, *tfull_bar = bars + 2 * DW_MAX_STAGES, *tempty_bar = tfull_bar + DW_ACC;
    uint32_t *tmem_slot = (uint32_t *)(tempty_bar + DW_ACC);
    int *slow_flag = (int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // a CTA keeps one channel group for its whole life, so its diagonal filter matrices are built once
    const int cg = blockIdx.x % p.ncg;
    const int tiles_per_cg = p.n * p.ytiles * p.xtiles;
    const int first_tile = blockIdx.x / p.ncg, tile_step = gridDim.x / p.ncg;
    const int c_base = cg * p.cg;
    const int cblocks = min(p.cg / 32, (p.c - c_base + 31) / 32);

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < DW_ACC; a++) {
            mbar_init(smem_u32(&tfull_bar[a]), 1);
            mbar_init(smem_u32(&tempty_bar[a]), 4);
        }
        *slow_flag = 0;
        fence_barrier_init();
    }
    // diag(w_tap) for this channel group: B[n][k], K-major, not swizzled: byte (n, k) at (k/16)*512 + n*16 + k%16
    for (int i = threadIdx.x; i < 4 * 9 * 1024 / 16; i += blockDim.x) ((uint4 *)b_smem)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    for (int i = threadIdx.x; i < 4 * 9 * 32; i += blockDim.x) {
        const int n = i % 32, tap = (i / 32) % 9, cb = i / (32 * 9);
        const int c = c_base + cb * 32 + n;
        if (c < p.c)
            b_smem[(cb * 9 + tap) * 1024 + (n / 16) * 512 + n * 16 + (n % 16)] = (uint8_t)p.w[(long long)tap * p.c + c];
    }
    // the unused tail of every stage is read by overhang rows only; whatever integers it holds end up in rows that are not stored
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 1)
        tmem_alloc(smem_u32(tmem_slot), 512);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const uint32_t tx = (uint32_t)(p.phases * p.cg * p.P * p.rows_in);
            for (int t = first_tile; t < tiles_per_cg && ok; t += tile_step) {
                const int xt = t % p.xtiles, yt = (t / p.xtiles) % p.ytiles, n = t / (p.xtiles * p.ytiles);
                if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1)) {
                    ok = false;
                    break;
                }
                const uint32_t bar = smem_u32(&full_bar[stage]);
                uint8_t *st = smem + (size_t)stage * stage_bytes;
                mbar_arrive_expect_tx(bar, tx);
                const int x0 = xt * p.two * p.S - p.pl, y0 = yt * p.R * p.S - p.pt;
                for (int ph = 0; ph < p.phases; ph++)
                    tma_load_4d(smem_u32(st + (size_t)ph * plane_bytes), &map_in, c_base, x0 + ph % p.S, y0 + ph / p.S, n, bar);
                if (++stage == p.stages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (!ok)
                atomicExch(&g_dw_tc_error, ESPDL_ERR_TIMEOUT);
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            const uint32_t idesc = idesc_i8(1, 1, 128, 32);
            for (int t = first_tile; t < tiles_per_cg && ok; t += tile_step) {
                if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1) || !mbar_wait(smem_u32(&full_bar[stage]), phase)) {
                    ok = false;
                    break;
                }
                fence_after();
                const uint32_t st = smem_u32(smem + (size_t)stage * stage_bytes);
                // Channel-block-major order: the nine taps of one accumulator are issued back to back (measured: alternating
                // accumulators between consecutive MMAs is 1.5x slower).  Each M=128 MMA occupies the pipe for about
                // 150 cycles whatever N is, which is what bounds this kernel (9 taps x 128 pixels x 32 channels each).
                for (int cb = 0; cb < cblocks; cb++) {
                    const uint32_t d = tmem_base + (uint32_t)(acc * DW_CG + cb * 32);
#pragma unroll
                    for (int tap = 0; tap < 9; tap++) {
                        const int ky = tap / 3, kx = tap % 3;
                        const int ph = (ky % p.S) * p.S + (kx % p.S);
                        const int off = (ky / p.S) * p.P + (kx / p.S);
                        // Row `off` of the plane, 32-byte channel block cb inside the row.  The swizzle is a function of
                        // the absolute shared-memory address (as for the TMA write), so a start address in the middle of
                        // the pattern needs nothing else: the descriptor's base-offset field stays 0 (measured: any
                        // other value breaks the 64- and 128-byte modes).
                        const uint32_t a_addr = st + (uint32_t)(ph * plane_bytes + off * p.cg + cb * 32);
                        const uint32_t b_addr = smem_u32(b_smem + (cb * 9 + tap) * 1024);
                        mma_i8(d, smem_desc_swizzled(a_addr, p.cg), smem_desc_plain(b_addr, 512, 128), idesc, tap != 0);
                    }
                }
                commit(smem_u32(&empty_bar[stage]));
                commit(smem_u32(&tfull_bar[acc]));
                if (++stage == p.stages) {
                    stage = 0;
                    phase ^= 1;
                }
                if (++acc == DW_ACC) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
            if (!ok)
                atomicExch(&g_dw_tc_error, ESPDL_ERR_TIMEOUT);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue: group g owns accumulator g
        const int acc = (warp - 2) >> 2;
        const int lane_group = warp & 3;
        const int m = lane_group * 32 + lane; // output pixel of the tile this thread owns
        const int ry = m / p.P, rx = m % p.P;
        const int et = threadIdx.x - 64;
        EpiConfig epi = p.epi;
        // channel-group view of the per-channel arrays
        if (epi.bias)
            epi.bias = (const int32_t *)epi.bias + c_base;
        if (epi.ew)
            epi.ew = epi.ew + c_base;
        const int n_valid = min(p.cg, p.c - c_base);
        stage_fast_params(epi, fast_s, n_valid, DW_CG, et, 16 * 32, slow_flag);
        asm volatile("bar.sync 1, %0;" ::"n"(16 * 32) : "memory");
        const bool fast = !*slow_flag && !epi.half_even && !epi.lut;
        uint32_t acc_phase = 0;
        bool ok = true;
        int local = 0;
        const bool vec_ok = (p.ops % 16 == 0) && ((((uintptr_t)p.out) + c_base) % 16 == 0);
        for (int t = first_tile; t < tiles_per_cg && ok; t += tile_step, local++) {
            if (local % DW_ACC != acc)
                continue;
            const int xt = t % p.xtiles, yt = (t / p.xtiles) % p.ytiles, n = t / (p.xtiles * p.ytiles);
            if (!mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase)) {
                ok = false;
                break;
            }
            acc_phase ^= 1;
            fence_after();
            const int oy = yt * p.R + ry, ox = xt * p.two + rx;
            const bool row_ok = ry < p.R && rx < p.two && oy < p.oh && ox < p.ow;
            int8_t *orow = (int8_t *)p.out + (((long long)n * p.oh + oy) * p.ow + ox) * p.ops + c_base;
            const uint32_t t0 = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(acc * DW_CG);
            for (int c0 = 0; c0 < cblocks * 32; c0 += 32) {
                int32_t v[32];
                ld16(t0 + c0, v);
                ld16(t0 + c0 + 16, v + 16);
                ld_wait16(v);
                tie16(v + 16);
                uint32_t pk[8];
                if (fast) {
                    if (epi.relu) {
                        requant16_fast<true>(v, fast_s + c0, pk);
                        requant16_fast<true>(v + 16, fast_s + c0 + 16, pk + 4);
                    } else {
                        requant16_fast<false>(v, fast_s + c0, pk);
                        requant16_fast<false>(v + 16, fast_s + c0 + 16, pk + 4);
                    }
                } else {
                    requant16_general(v, epi, c0, n_valid, pk);
                    requant16_general(v + 16, epi, c0 + 16, n_valid, pk + 4);
                }
                if (row_ok) {
                    const int count = min(32, n_valid - c0);
                    if (count > 0)
                        store_bytes(orow + c0, pk, count, vec_ok ? 16 : 1);
                }
            }
            fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(smem_u32(&tempty_bar[acc]));
        }
        if (!ok && lane == 0)
            atomicExch(&g_dw_tc_error, ESPDL_ERR_TIMEOUT);
    }

    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_dw()
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

constexpr size_t DW_SMEM_BUDGET = 200 * 1024;

bool plan_dw(const espdl_conv_desc &d, DwTcParams &p)
{
    p.n = d.n, p.ih = d.in_h, p.iw = d.in_w, p.c = d.in_c, p.oh = d.out_h, p.ow = d.out_w;
    p.S = d.stride_h, p.pt = d.pad_top, p.pl = d.pad_left;
    p.phases = p.S * p.S;
    // pitch 16 or 32: whichever wastes fewer of the 128 rows of a tile
    double best = -1;
    for (int P : {16, 32}) {
        const int two = P - (p.S == 1 ? 2 : 1), R = 128 / P;
        const int xt = (d.out_w + two - 1) / two, yt = (d.out_h + R - 1) / R;
        const double eff = (double)d.out_w * d.out_h / ((double)xt * yt * 128);
        if (eff > best) {
            best = eff;
            p.P = P, p.R = R, p.two = two, p.xtiles = xt, p.ytiles = yt;
        }
    }
    p.rows_in = p.R + (p.S == 1 ? 2 : 1);
    p.plane_px = (p.rows_in + 1) * p.P; // one slack row: overhang rows of the MMA read past the loaded window
    p.cg = d.in_c >= 128 ? 128 : (d.in_c >= 64 ? 64 : 32);
    if (p.S == 2 && p.cg > 64)
        p.cg = 64; // four parity planes per stage: 64-byte rows keep three stages in shared memory
    p.ncg = (d.in_c + p.cg - 1) / p.cg;
    const size_t stage_bytes = (size_t)p.phases * p.plane_px * p.cg;
    const size_t aux = 4 * 9 * 1024 + sizeof(FastParam) * DW_CG + (2 * DW_MAX_STAGES + 2 * DW_ACC) * 8 + 32;
    int stages = (int)((DW_SMEM_BUDGET - aux - 2048) / stage_bytes);
    if (stages < 2)
        return false;
    p.stages = min(stages, DW_MAX_STAGES);
    return p.ncg <= num_sms();
}

} // namespace

bool conv2d_dw_tc_supported(const espdl_conv_desc &d)
{
    if (d.dtype != ESPDL_DTYPE_INT8 || d.group == 1 || d.kh != 3 || d.kw != 3 || d.dilation_h != 1 || d.dilation_w != 1)
        return false;
    if (d.stride_h != d.stride_w || (d.stride_h != 1 && d.stride_h != 2))
        return false;
    const int ips = d.in_pixel_stride ? d.in_pixel_stride : d.in_c;
    if (d.in_c % 16 || ips % 16 || ((uintptr_t)d.input % 16))
        return false;
    if (d.pad_top > 2 || d.pad_left > 2 || (long long)d.n * d.in_h * d.in_w * ips > 0x7fffffffffll)
        return false;
    DwTcParams p;
    return plan_dw(d, p);
}

int conv2d_dw_tc(const espdl_conv_desc &d, cudaStream_t s)
{
    DwTcParams p;
    if (!plan_dw(d, p))
        return ESPDL_ERR_UNSUPPORTED;
    const int ips = d.in_pixel_stride ? d.in_pixel_stride : d.in_c;
    p.ops = d.out_pixel_stride ? d.out_pixel_stride : d.out_c;
    p.out = d.output, p.w = (const int8_t *)d.filter;
    p.epi.bias = d.bias, p.epi.ew = d.filter_exponents, p.epi.lut = d.lut;
    p.epi.e_shift_base = d.out_exponent - d.in_exponent;
    p.epi.ew_scalar = d.filter_exponent, p.epi.per_channel = d.per_channel;
    p.epi.relu = d.activation == ESPDL_ACT_RELU, p.epi.half_even = d.round_mode == ESPDL_ROUND_HALF_EVEN;

    EncodeTiledFn enc = get_encode_dw();
    if (!enc)
        return set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point not found");
    CUtensorMap map;
    cuuint64_t dims[4] = {(cuuint64_t)d.in_c, (cuuint64_t)d.in_w, (cuuint64_t)d.in_h, (cuuint64_t)d.n};
    cuuint64_t strides[3] = {(cuuint64_t)ips, (cuuint64_t)ips * d.in_w, (cuuint64_t)ips * d.in_w * d.in_h};
    cuuint32_t box[4] = {(cuuint32_t)p.cg, (cuuint32_t)(p.P * p.S), (cuuint32_t)(p.rows_in * p.S), 1};
    const CUtensorMapSwizzle sw = p.cg == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (p.cg == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    cuuint32_t estr[4] = {1, (cuuint32_t)p.S, (cuuint32_t)p.S, 1};
    CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(d.input), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(depthwise)");

    const size_t stage_bytes = (size_t)p.phases * p.plane_px * p.cg;
    const size_t smem = 1024 + (size_t)p.stages * stage_bytes + 4 * 9 * 1024 + sizeof(FastParam) * DW_CG + (2 * DW_MAX_STAGES + 2 * DW_ACC) * 8 + 32 +
        1024;
    static std::once_flag attr_once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(attr_once, [] {
        attr_err = cudaFuncSetAttribute(dw_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(DW_SMEM_BUDGET + 4096));
    });
    if (attr_err != cudaSuccess)
        return set_cuda_error(attr_err, "cudaFuncSetAttribute(dw_tc_kernel)");
    const long long tiles = (long long)p.n * p.ytiles * p.xtiles;
    int per_cg = (int)min((long long)(num_sms() / p.ncg), tiles);
    if (per_cg < 1)
        per_cg = 1;
    const int grid = per_cg * p.ncg;
    dw_tc_kernel<<<grid, DW_THREADS, max(smem, (size_t)120 * 1024), s>>>(map, p);
    count_launch();
    return check_launch("dw_tc");
}

} // namespace espdl
