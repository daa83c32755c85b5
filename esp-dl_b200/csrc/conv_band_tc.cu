// 3x3 convolutions with few input channels (8 or 16) on the tensor cores, stride 1 or 2, int8.
//
// With Cin = 8 or 16 a tap holds 8 or 16 bytes of reduction: the implicit-GEMM tile kernel would move 16-byte rows
// through the TMA unit and issue MMAs of N = Cout <= 32, a few per cent of what the tensor pipe and the TMA unit can do
// (measured on the detector's first layers: 2.1-3.1 ms for convolutions whose tensors take 50-190 us to move).  Here the
// reduction runs over a contiguous 128-byte piece of an input ROW, as in the first-layer kernel (stem_tc.cu): J
// neighbouring outputs of one output row read the same window of 128 / Cin input pixels of each of their three input
// rows, and the filter becomes three banded planes
//
//     D[(image, y), (j, co)] = sum_ky sum_k  A_ky[(image, y), k] * B_ky[(j, co), k]          j = 0..J-1, k = 0..127
//     A_ky[(image, y), k]    = byte k of the window of input row S*y + ky - pad_top that starts at pixel J*S*s - shift
//     B_ky[(j, co), k]       = w[co][ky][kx][c]  where  k = k_base + S*Cin*j + Cin*kx + c    (zero elsewhere)
//
// built once per CTA in shared memory.  A needs no gathering: one 3-D TMA box {128 bytes, rows_y output rows, rows_n
// images} per ky, of a tensor map whose row dimension steps S input rows, lands as the K-major 128-byte-swizzled operand;
// rows and bytes outside the image arrive as zeros (the padding rule of esp-dl/dl/base/dl_base.hpp:1209-2107).  Twelve
// MMAs (3 ky x 4 x K = 32) produce a tile of 128 (image, y) rows x J outputs x Cout channels; a tile row is J * Cout
// contiguous bytes of the NHWC output.  J is the largest count for which the window holds every tap, J * Cout fills whole
// 32-column halves of at most 256 accumulator columns, and the window starts on a 16-byte boundary.
//
// Replaces dl::base::conv2d<int8_t,...> (esp-dl/dl/base/dl_base_conv2d.cpp:9-60) for these shapes.  Roles, barriers and
// bounded waits are those of the pointwise tile kernel (gemm_tc.cu).
#include "tc_common.cuh"

#include <mutex>

namespace espdl {

__device__ int g_band_tc_error = 0;

int read_and_clear_device_error_band()
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_band_tc_error, sizeof(int)) != cudaSuccess)
        return 0;
    if (v) {
        int zero = 0;
        cudaMemcpyToSymbol(g_band_tc_error, &zero, sizeof(int));
    }
    return v;
}

namespace {

using namespace tc;

constexpr int BD_THREADS = 64 + 16 * 32; // TMA warp, MMA warp, 16 epilogue warps
constexpr int BD_K = 128;                // bytes of an input row per tile row
constexpr int BD_ACC = 2;
constexpr int BD_A_BYTES = 128 * BD_K;   // one ky plane of a stage
constexpr int BD_MAX_STAGES = 4;

struct BandParams {
    int n, ih, iw, oh, ow, cin, cout, S, J;
    int ncol, out_pw, out_mask; // accumulator columns J * Cout; a group's piece = half of them; swizzle mask of the staging tile
    int stages;
    int rows_n, rows_y;      // tile rows = rows_n images x rows_y output rows = 128
    int segs, yblocks, ngroups;
    int seg_bytes;           // J * S * Cin: input bytes between neighbouring windows
    int x_shift, k_base;     // window start = seg_bytes*s - x_shift; tap (j, kx, c) sits at byte k_base + S*Cin*j + Cin*kx + c
    int yq[3];               // TMA row coordinate of output row y for filter row ky: y + yq[ky]
    const int8_t *w;         // [Cout][3][3][Cin]
    void *out;
    EpiConfig epi;
};

__global__ void __launch_bounds__(BD_THREADS, 1)
band_tc_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1, const __grid_constant__ CUtensorMap map2,
               const __grid_constant__ CUtensorMap map_out, const __grid_constant__ BandParams p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int ncol = p.ncol;                                    // accumulator columns = B rows (<= 256, multiple of 32)
    const int b_plane = ((ncol * BD_K) + 1023) & ~1023;         // one ky plane of B
    uint8_t *b_s = smem;                                        // 3 planes
    uint8_t *a_s = smem + 3 * (size_t)b_plane;                  // stages x 3 planes
    uint8_t *out_stage = a_s + (size_t)p.stages * 3 * BD_A_BYTES; // four [128][out_pw] byte tiles, one per epilogue group
    const int out_pw = p.out_pw;
    const int out_tile_bytes = (128 * out_pw + 1023) & ~1023;
    uint8_t *aux = out_stage + 4 * (size_t)out_tile_bytes;
    FastParam *fast_s = (FastParam *)aux;                       // one entry per accumulator column
    uint64_t *bars = (uint64_t *)(aux + sizeof(FastParam) * 256);
    uint64_t *full_bar = bars, *empty_bar = bars + BD_MAX_STAGES, *tfull_bar = bars + 2 * BD_MAX_STAGES, *tempty_bar = tfull_bar + BD_ACC;
    uint32_t *tmem_slot = (uint32_t *)(tempty_bar + BD_ACC);
    int *slow_flag = (int *)(tmem_slot + 1);
    uint8_t *lut_s = (uint8_t *)(slow_flag + 3); // a fused 8-bit table, 256 bytes, 16-byte aligned

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = p.ngroups * p.yblocks * p.segs;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < BD_ACC; a++) {
            mbar_init(smem_u32(&tfull_bar[a]), 1);
            mbar_init(smem_u32(&tempty_bar[a]), 8); // the two groups of four warps that share an accumulator
        }
        *slow_flag = 0;
        fence_barrier_init();
    }
    // banded filter planes, written in the 128-byte-swizzled K-major layout the MMA reads: the 16-byte chunk index of a
    // row is XORed with bits 7-9 of the byte offset (planes start on 1024-byte boundaries)
    {
        const int words_per_plane = ncol * (BD_K / 4);
        const int tap_bytes = 3 * p.cin, step = p.S * p.cin;
        for (int i = threadIdx.x; i < 3 * words_per_plane; i += BD_THREADS) {
            const int ky = i / words_per_plane, r = i - ky * words_per_plane;
            const int row = r >> 5, k0 = (r & 31) * 4;
            const int j = row / p.cout, co = row - j * p.cout;
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; b++) {
                const int t = k0 + b - p.k_base - step * j; // Cin*kx + c
                if (t >= 0 && t < tap_bytes)
                    word |= (uint32_t)(uint8_t)p.w[(co * 3 + ky) * tap_bytes + t] << (8 * b);
            }
            const uint32_t off = (uint32_t)(row * BD_K + k0);
            *(uint32_t *)(b_s + (size_t)ky * b_plane + (off ^ (((off >> 7) & 7u) << 4))) = word;
        }
    }
    if (p.epi.lut)
        stage_lut(p.epi.lut, lut_s, (int)threadIdx.x, BD_THREADS);
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
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int s = tile % p.segs;
                const int yb = (tile / p.segs) % p.yblocks;
                const int ng = tile / (p.segs * p.yblocks);
                if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1)) {
                    ok = false;
                    break;
                }
                const uint32_t bar = smem_u32(&full_bar[stage]);
                uint8_t *st = a_s + (size_t)stage * 3 * BD_A_BYTES;
                mbar_arrive_expect_tx(bar, 3u * BD_A_BYTES);
                const int x = p.seg_bytes * s - p.x_shift, y = yb * p.rows_y, n0 = ng * p.rows_n; // x is a multiple of 16
                tma_load_3d(smem_u32(st), &map0, x, y + p.yq[0], n0, bar);
                tma_load_3d(smem_u32(st + BD_A_BYTES), &map1, x, y + p.yq[1], n0, bar);
                tma_load_3d(smem_u32(st + 2 * BD_A_BYTES), &map2, x, y + p.yq[2], n0, bar);
                if (++stage == p.stages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (!ok)
                atomicExch(&g_band_tc_error, ESPDL_ERR_TIMEOUT);
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            const uint32_t idesc = idesc_i8(1, 1, 128, ncol);
            const uint32_t b0 = smem_u32(b_s);
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1) || !mbar_wait(smem_u32(&full_bar[stage]), phase)) {
                    ok = false;
                    break;
                }
                fence_after();
                const uint32_t d0 = tmem_base + (uint32_t)(acc * 256);
                const uint32_t st = smem_u32(a_s + (size_t)stage * 3 * BD_A_BYTES);
#pragma unroll
                for (int ky = 0; ky < 3; ky++) {
                    const uint64_t da = smem_desc_swizzled(st + ky * BD_A_BYTES, 128);
                    const uint64_t db = smem_desc_swizzled(b0 + ky * b_plane, 128);
                    mma_i8(d0, da, db, idesc, ky != 0);
                    mma_i8(d0, da + 2, db + 2, idesc, 1u); // the next 32 bytes of K
                    mma_i8(d0, da + 4, db + 4, idesc, 1u);
                    mma_i8(d0, da + 6, db + 6, idesc, 1u);
                }
                commit(smem_u32(&empty_bar[stage]));
                commit(smem_u32(&tfull_bar[acc]));
                if (++stage == p.stages) {
                    stage = 0;
                    phase ^= 1;
                }
                if (++acc == BD_ACC) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
            if (!ok)
                atomicExch(&g_band_tc_error, ESPDL_ERR_TIMEOUT);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..17)
        const int ew = warp - 2;
        const int group = ew >> 2;       // 0..3
        const int acc = group % BD_ACC;  // accumulator buffer this group reads
        const int part = group / BD_ACC; // which half of the tile's columns
        const int lane_group = warp & 3;
        const int row_in_tile = lane_group * 32 + lane;
        const int et = threadIdx.x - 64;
        // constants of the one-add-one-shift form per accumulator column (column = j * Cout + channel)
        {
            int bad = 0;
            for (int col = et; col < 256; col += 16 * 32) {
                int b = 0, sh = 1;
                if (col < ncol) {
                    const int c = col % p.cout;
                    if (p.epi.bias)
                        b = ((const int32_t *)p.epi.bias)[c];
                    sh = p.epi.e_shift_base - (p.epi.per_channel ? p.epi.ew[c] : p.epi.ew_scalar);
                    if (sh < 1 || sh > 24 || b >= (1 << 30) || b <= -(1 << 30))
                        bad = 1;
                    sh = max(1, min(24, sh));
                }
                fast_s[col].bias_half = b + (1 << (sh - 1));
                fast_s[col].shift = sh;
            }
            if (bad)
                atomicOr(slow_flag, 1);
        }
        asm volatile("bar.sync 1, %0;" ::"n"(16 * 32) : "memory");
        const bool fast = !*slow_flag && !p.epi.half_even && !p.epi.lut_stride; // one fused table rides on the staged form, per-channel tables take the general path
        const uint32_t fp = epi_param_base(fast_s);
        uint32_t acc_phase = 0;
        bool ok = true;
        int local = 0;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, local++) {
            if (local % BD_ACC != acc)
                continue;
            const int s = tile % p.segs;
            const int yb = (tile / p.segs) % p.yblocks;
            const int ng = tile / (p.segs * p.yblocks);
            if (!mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase)) {
                ok = false;
                break;
            }
            acc_phase ^= 1;
            fence_after();
            const int n = ng * p.rows_n + row_in_tile / p.rows_y;
            const int y = yb * p.rows_y + row_in_tile % p.rows_y;
            const bool row_ok = n < p.n && y < p.oh;
            const int ncols = min(p.J, p.ow - p.J * s) * p.cout;
            int8_t *orow = (int8_t *)p.out + (((long long)n * p.oh + y) * p.ow + p.J * s) * p.cout;
            const uint32_t t0 = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(acc * 256);
            if (fast) {
                // rows are requantised into this group's shared-memory tile and leave through one 3-D TMA store,
                // which also clips the ragged last group of outputs and rows outside the image
                const bool leader = (ew & 3) == 0 && lane == 0;
                const uint32_t buf = smem_u32(out_stage + (size_t)group * out_tile_bytes);
                if (leader)
                    bulk_wait_read_all();
                named_bar(2 + group, 128);
                const int col0 = part * out_pw;
                const int floor_q = p.epi.relu ? 0 : INT_MIN;
                if (p.epi.lut)
                    epilogue_stage_lut(t0 + col0, fp + (uint32_t)col0 * 8u, buf, row_in_tile, out_pw, (uint32_t)p.out_mask, floor_q, smem_u32(lut_s));
                else if (out_pw == 128)
                    epilogue_stage<128>(t0 + col0, fp + (uint32_t)col0 * 8u, buf, row_in_tile, 128, floor_q);
                else if (out_pw == 64)
                    epilogue_stage<64>(t0 + col0, fp + (uint32_t)col0 * 8u, buf, row_in_tile, 64, floor_q);
                else
                    epilogue_stage<0>(t0 + col0, fp + (uint32_t)col0 * 8u, buf, row_in_tile, out_pw, floor_q);
                fence_before();
                fence_async_smem();
                named_bar(2 + group, 128);
                if (leader) {
                    tma_store_3d(&map_out, buf, p.J * s * p.cout + col0, yb * p.rows_y, ng * p.rows_n);
                    bulk_commit();
                }
            } else {
                int chunk = 0;
                for (int c0 = 0; c0 < ncol; c0 += 16, chunk++) {
                    if ((c0 >= out_pw ? 1 : 0) != part)
                        continue;
                    int32_t v[16];
                    ld16(t0 + c0, v);
                    ld_wait16(v);
                    uint32_t pk[4] = {0, 0, 0, 0};
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const int c = (c0 + i) % p.cout;
                        const int e = p.epi.per_channel ? __ldg(p.epi.ew + c) : p.epi.ew_scalar;
                        const int shift = max(-31, min(31, p.epi.e_shift_base - e));
                        int32_t r = requant8(v[i], p.epi.bias ? __ldg((const int32_t *)p.epi.bias + c) : 0, shift, p.epi.relu, p.epi.half_even);
                        if (p.epi.lut)
                            r = p.epi.lut[(long long)c * p.epi.lut_stride + ((uint8_t)r ^ 0x80u)];
                        pk[i >> 2] |= ((uint32_t)r & 0xffu) << (8 * (i & 3));
                    }
                    // whole 16-byte groups only when the row's bytes are aligned; otherwise byte by byte
                    if (row_ok && c0 < ncols) {
                        if (c0 + 16 <= ncols && ((((uintptr_t)(orow + c0))) & 15) == 0) {
                            *(uint4 *)(orow + c0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                        } else {
                            for (int i = 0; i < 16 && c0 + i < ncols; i++) orow[c0 + i] = (int8_t)(pk[i >> 2] >> (8 * (i & 3)));
                        }
                    }
                }
            }
            fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(smem_u32(&tempty_bar[acc]));
        }
        if (!ok && lane == 0)
            atomicExch(&g_band_tc_error, ESPDL_ERR_TIMEOUT);
        if ((ew & 3) == 0 && lane == 0)
            bulk_wait_all(); // shared memory stays allocated until the last store has left it
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

EncodeTiledFn band_encode()
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

// Outputs per window (0 = this shape is not taken) and where the window starts relative to the first output's first tap.
// The window holds 128 / Cin pixels and starts `shift_px` pixels left of pixel J*S*s (a 16-byte boundary); output j reads
// pixels J*S*s - pad_left + S*j + {0, 1, 2}.
size_t band_fixed_smem(int ncol)
{
    const size_t b_plane = ((size_t)ncol * BD_K + 1023) & ~(size_t)1023;
    const size_t out_tile = ((size_t)128 * (ncol / 2) + 1023) & ~(size_t)1023;
    return 1024 + 3 * b_plane + 4 * out_tile + sizeof(FastParam) * 256 + (2 * BD_MAX_STAGES + 2 * BD_ACC) * 8 + 64 + 256;
}
constexpr size_t BD_SMEM_BUDGET = 220 * 1024;

int band_outputs(const espdl_conv_desc &d, int &shift_px)
{
    const int px = BD_K / d.in_c, S = d.stride_w;
    const int align_px = 16 / d.in_c > 1 ? 16 / d.in_c : 1; // pixels per 16 bytes (2 for Cin = 8)
    shift_px = d.pad_left ? ((d.pad_left + align_px - 1) / align_px) * align_px : 0;
    int best = 0;
    for (int J = 1; J <= 16; J++) {
        if ((J * S) % align_px != 0)
            continue; // the next window would not start on a 16-byte boundary
        const int last_px = shift_px - d.pad_left + S * (J - 1) + 2; // last pixel of the window any tap of output J-1 reads
        if (last_px >= px)
            break;
        const int ncol = J * d.out_c;
        if (ncol > 256 || ncol % 32 != 0)
            continue;
        if (band_fixed_smem(ncol) + 2 * 3 * (size_t)BD_A_BYTES > BD_SMEM_BUDGET)
            continue; // no room for two stages of input planes next to this many filter rows
        best = J;
    }
    return best;
}

} // namespace

bool conv2d_band_tc_supported(const espdl_conv_desc &d)
{
    if (getenv("ESPDL_B200_NO_BAND_CONV"))
        return false;
    if (d.dtype != ESPDL_DTYPE_INT8 || d.group != 1 || d.kh != 3 || d.kw != 3 || (d.in_c != 8 && d.in_c != 16))
        return false;
    if (d.stride_h != d.stride_w || (d.stride_h != 1 && d.stride_h != 2) || d.dilation_h != 1 || d.dilation_w != 1)
        return false;
    if (d.pad_top < 0 || d.pad_top > 1 || d.pad_left < 0 || d.pad_left > 1 || d.residual || d.filter_image_stride)
        return false;
    if (d.out_c % 8 != 0 || d.out_c > 64)
        return false;
    if ((d.in_pixel_stride && d.in_pixel_stride != d.in_c) || (d.out_pixel_stride && d.out_pixel_stride != d.out_c))
        return false;
    const long long row_bytes = (long long)d.in_c * d.in_w, out_row_bytes = (long long)d.out_c * d.out_w;
    if (row_bytes % 16 != 0 || out_row_bytes % 16 != 0 || ((uintptr_t)d.input % 16) || ((uintptr_t)d.output % 16) || d.in_h < 3)
        return false;
    int shift_px;
    const int J = band_outputs(d, shift_px);
    // a piece of J * Cout / 2 bytes must start on a 16-byte boundary of the output row for the TMA store
    return J > 0 && (J * d.out_c / 2) % 16 == 0;
}

int conv2d_band_tc(const espdl_conv_desc &d, cudaStream_t s)
{
    if (!conv2d_band_tc_supported(d))
        return ESPDL_ERR_UNSUPPORTED;
    EncodeTiledFn enc = band_encode();
    if (!enc)
        return set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point not found");
    BandParams p;
    memset(&p, 0, sizeof(p));
    int shift_px = 0;
    p.J = band_outputs(d, shift_px);
    p.n = d.n, p.ih = d.in_h, p.iw = d.in_w, p.oh = d.out_h, p.ow = d.out_w, p.cin = d.in_c, p.cout = d.out_c, p.S = d.stride_w;
    p.ncol = p.J * d.out_c, p.out_pw = p.ncol / 2;
    p.out_mask = p.out_pw == 128 ? 7 : (p.out_pw == 64 ? 3 : 0);
    p.rows_n = d.n >= 8 ? 8 : (d.n >= 4 ? 4 : (d.n >= 2 ? 2 : 1));
    p.rows_y = 128 / p.rows_n;
    p.segs = (d.out_w + p.J - 1) / p.J;
    p.yblocks = (d.out_h + p.rows_y - 1) / p.rows_y;
    p.ngroups = (d.n + p.rows_n - 1) / p.rows_n;
    p.seg_bytes = p.J * p.S * d.in_c;
    p.x_shift = shift_px * d.in_c;
    p.k_base = (shift_px - d.pad_left) * d.in_c;
    p.w = (const int8_t *)d.filter, p.out = d.output;
    p.epi.bias = d.bias, p.epi.ew = d.filter_exponents, p.epi.lut = d.lut, p.epi.lut_stride = d.lut_channel_stride;
    p.epi.e_shift_base = d.out_exponent - d.in_exponent;
    p.epi.ew_scalar = d.filter_exponent, p.epi.per_channel = d.per_channel;
    p.epi.relu = d.activation == ESPDL_ACT_RELU, p.epi.half_even = d.round_mode == ESPDL_ROUND_HALF_EVEN;

    // shared memory: three filter planes, the staging tiles, and as many stages of three input planes as fit
    const size_t fixed = band_fixed_smem(p.ncol);
    p.stages = (int)min((size_t)BD_MAX_STAGES, (BD_SMEM_BUDGET - fixed) / (3 * (size_t)BD_A_BYTES));
    if (p.stages < 2)
        return ESPDL_ERR_UNSUPPORTED;

    // One map per filter row ky: input rows S*y + ky - pad_top = S*(y + q) + r, so the map starts at row r, steps S rows
    // per index and is addressed with y + q; indices outside [0, rows of that phase) read zeros.
    CUtensorMap maps[3];
    const uint64_t row_bytes = (uint64_t)d.in_c * d.in_w;
    for (int ky = 0; ky < 3; ky++) {
        const int off = ky - d.pad_top;
        const int r = ((off % p.S) + p.S) % p.S, q = (off - r) / p.S;
        p.yq[ky] = q;
        cuuint64_t dims[3] = {row_bytes, (cuuint64_t)((d.in_h - r + p.S - 1) / p.S), (cuuint64_t)d.n};
        cuuint64_t strides[2] = {(cuuint64_t)p.S * row_bytes, (cuuint64_t)d.in_h * row_bytes};
        cuuint32_t box[3] = {BD_K, (cuuint32_t)p.rows_y, (cuuint32_t)p.rows_n};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult res = enc(&maps[ky], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, (void *)((const uint8_t *)d.input + r * row_bytes), dims, strides, box,
                           estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (res != CUDA_SUCCESS)
            return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(band conv input)");
    }
    // output as a 3-D tensor {OW*Cout bytes, OH, N}; a group's piece is half of a tile row
    CUtensorMap mo;
    {
        cuuint64_t dims[3] = {(cuuint64_t)d.out_w * d.out_c, (cuuint64_t)d.out_h, (cuuint64_t)d.n};
        cuuint64_t strides[2] = {(cuuint64_t)d.out_w * d.out_c, (cuuint64_t)d.out_h * d.out_w * d.out_c};
        cuuint32_t box[3] = {(cuuint32_t)p.out_pw, (cuuint32_t)p.rows_y, (cuuint32_t)p.rows_n};
        cuuint32_t estr[3] = {1, 1, 1};
        const CUtensorMapSwizzle sw = p.out_pw == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (p.out_pw == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE);
        if (enc(&mo, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, d.output, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(band conv output)");
    }
    const size_t smem = fixed + (size_t)p.stages * 3 * BD_A_BYTES;
    static std::once_flag attr_once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(attr_once, [] { attr_err = cudaFuncSetAttribute(band_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024); });
    if (attr_err != cudaSuccess)
        return set_cuda_error(attr_err, "cudaFuncSetAttribute(band_tc_kernel)");
    const int total = p.ngroups * p.yblocks * p.segs;
    const int grid = min(total, num_sms());
    band_tc_kernel<<<grid, BD_THREADS, max(smem, (size_t)120 * 1024), s>>>(maps[0], maps[1], maps[2], mo, p);
    count_launch();
    return check_launch("band_tc");
}

} // namespace espdl
