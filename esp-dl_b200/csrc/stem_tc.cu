// First layer of an image network on the tensor cores: 3x3 conv, stride 2, 3 input channels (RGB), int8.
//
// With Cin = 3 the reduction length of a pixel is 27: far too short for an implicit-GEMM tile, and gathering 27
// bytes per pixel costs more than the arithmetic.  Here the reduction runs over a contiguous piece of an input
// ROW instead.  Eight neighbouring outputs of one output row read input bytes [48*s - a, 48*s - a + 64) of each of
// their three input rows (s = index of the group of eight, a = 16 when there is left padding, else 0):
//
//     D[(image, y), (j, co)] = sum_ky sum_k  A_ky[(image, y), k] * B_ky[(j, co), k]          j = 0..7, k = 0..63
//     A_ky[(image, y), k]    = byte k of that 64-byte window of input row 2*y + ky - pad_top
//     B_ky[(j, co), k]       = w[co][ky][kx][c]  where  k = base + 6*j + 3*kx + c   (zero elsewhere)
//
// B is a banded ("Toeplitz") copy of the 3x3x3 filter, 8*Cout rows of 64 bytes per ky, built once per CTA in
// shared memory.  A needs no gathering at all: one 3-D TMA box {64 bytes, rows_y output rows, rows_n images} of a
// tensor map whose row dimension steps by two input rows lands in shared memory as the K-major swizzled operand,
// 128 rows of 64 bytes.  Rows above or below the image, bytes left of its first or right of its last pixel are
// outside the tensor map and arrive as zeros, which is the padding rule of esp-dl/dl/base/dl_base.hpp:1209-2107.
// Six MMAs (3 ky x K = 2 x 32) produce a tile of 128 (image, y) rows x 8 outputs x Cout channels, and a tile row
// is 8 * Cout CONTIGUOUS bytes of the NHWC output, written by the tile kernels' lean epilogue.
//
// Replaces dl::base::conv2d<int8_t,...> (esp-dl/dl/base/dl_base_conv2d.cpp:9-60) for this shape.  Roles, barriers
// and bounded waits are those of the pointwise tile kernel (gemm_tc.cu).
#include "tc_common.cuh"

#include <mutex>

namespace espdl {

__device__ int g_stem_tc_error = 0;

int read_and_clear_device_error_stem()
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_stem_tc_error, sizeof(int)) != cudaSuccess)
        return 0;
    if (v) {
        int zero = 0;
        cudaMemcpyToSymbol(g_stem_tc_error, &zero, sizeof(int));
    }
    return v;
}

namespace {

using namespace tc;

constexpr int ST_THREADS = 64 + 16 * 32; // TMA warp, MMA warp, 16 epilogue warps
constexpr int ST_J = 8;                  // outputs of one row per tile row
constexpr int ST_K = 64;                 // bytes of an input row per tile row
constexpr int ST_STAGES = 4;
constexpr int ST_ACC = 2;
constexpr int ST_A_BYTES = 128 * ST_K;   // one ky plane of a stage

struct StemParams {
    int n, ih, iw, oh, ow, cout;
    int pt, pl;
    int rows_n, rows_y;      // tile rows = rows_n images x rows_y output rows = 128
    int segs, yblocks, ngroups;
    int x_shift, k_base;     // window start = 48*s - x_shift; tap (j, kx, c) sits at byte k_base + 6*j + 3*kx + c
    int yq[3];               // TMA row coordinate of output row y for filter row ky: y + yq[ky]
    const int8_t *w;
    void *out;
    EpiConfig epi;
};

__global__ void __launch_bounds__(ST_THREADS, 1)
stem_tc_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1, const __grid_constant__ CUtensorMap map2,
               const __grid_constant__ CUtensorMap map_out, const StemParams p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int ncol = ST_J * p.cout;            // accumulator columns = B rows (<= 256, multiple of 16)
    const int b_bytes = ncol * ST_K;           // one ky plane of B
    uint8_t *b_s = smem;                                        // 3 planes
    uint8_t *a_s = smem + 3 * 256 * ST_K;                       // stages x 3 planes
    uint8_t *out_stage = a_s + ST_STAGES * 3 * ST_A_BYTES;      // four [128][ncol/2] byte tiles, one per epilogue group
    const int out_pw = ncol / 2;
    const int out_tile_bytes = 128 * out_pw;
    uint8_t *aux = out_stage + 4 * 128 * 128;
    FastParam *fast_s = (FastParam *)aux;                       // one entry per accumulator column
    uint64_t *bars = (uint64_t *)(aux + sizeof(FastParam) * 256);
    uint64_t *full_bar = bars, *empty_bar = bars + ST_STAGES, *tfull_bar = bars + 2 * ST_STAGES, *tempty_bar = tfull_bar + ST_ACC;
    uint32_t *tmem_slot = (uint32_t *)(tempty_bar + ST_ACC);
    int *slow_flag = (int *)(tmem_slot + 1);
    uint8_t *lut_s = (uint8_t *)(slow_flag + 3); // a fused 8-bit table, 256 bytes, 16-byte aligned

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = p.ngroups * p.yblocks * p.segs;

    if (threadIdx.x == 0) {
        for (int s = 0; s < ST_STAGES; s++) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < ST_ACC; a++) {
            mbar_init(smem_u32(&tfull_bar[a]), 1);
            mbar_init(smem_u32(&tempty_bar[a]), 8); // the two groups of four warps that share an accumulator
        }
        *slow_flag = 0;
        fence_barrier_init();
    }
    // banded filter planes, written in the 64-byte-swizzled K-major layout the MMA reads: the 16-byte chunk index
    // of a row is XORed with bits 7-8 of the byte offset (planes start on 1024-byte boundaries)
    const int cout_log2 = p.cout == 32 ? 5 : 4; // Cout is 16 or 32: shifts instead of divisions
    for (int i = threadIdx.x; i < 3 * 256 * (ST_K / 4); i += ST_THREADS) {
        const int ky = i >> 12;                 // 256 rows x 16 words per plane
        const int row = (i >> 4) & 255, k0 = (i & 15) * 4;
        if (row >= ncol)
            continue;
        const int j = row >> cout_log2, co = row & (p.cout - 1);
        uint32_t word = 0;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const int t = k0 + b - p.k_base - 6 * j; // 3*kx + c
            if (t >= 0 && t < 9)
                word |= (uint32_t)(uint8_t)p.w[(co * 3 + ky) * 9 + t] << (8 * b);
        }
        const uint32_t off = (uint32_t)(row * ST_K + k0);
        *(uint32_t *)(b_s + (size_t)ky * 256 * ST_K + (off ^ (((off >> 7) & 3u) << 4))) = word;
    }
    if (p.epi.lut)
        stage_lut(p.epi.lut, lut_s, (int)threadIdx.x, ST_THREADS);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 1)
        tmem_alloc(smem_u32(tmem_slot), 512);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = *tmem_slot;
    (void)b_bytes;

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
                uint8_t *st = a_s + (size_t)stage * 3 * ST_A_BYTES;
                mbar_arrive_expect_tx(bar, 3u * ST_A_BYTES);
                const int x = 6 * ST_J * s - p.x_shift, y = yb * p.rows_y, n0 = ng * p.rows_n;
                tma_load_3d(smem_u32(st), &map0, x, y + p.yq[0], n0, bar);
                tma_load_3d(smem_u32(st + ST_A_BYTES), &map1, x, y + p.yq[1], n0, bar);
                tma_load_3d(smem_u32(st + 2 * ST_A_BYTES), &map2, x, y + p.yq[2], n0, bar);
                if (++stage == ST_STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (!ok)
                atomicExch(&g_stem_tc_error, ESPDL_ERR_TIMEOUT);
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
                const uint32_t st = smem_u32(a_s + (size_t)stage * 3 * ST_A_BYTES);
#pragma unroll
                for (int ky = 0; ky < 3; ky++) {
                    const uint64_t da = smem_desc_swizzled(st + ky * ST_A_BYTES, 64);
                    const uint64_t db = smem_desc_swizzled(b0 + ky * 256 * ST_K, 64);
                    mma_i8(d0, da, db, idesc, ky != 0);
                    mma_i8(d0, da + 2, db + 2, idesc, 1u); // next 32 bytes of K
                }
                commit(smem_u32(&empty_bar[stage]));
                commit(smem_u32(&tfull_bar[acc]));
                if (++stage == ST_STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
                if (++acc == ST_ACC) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
            if (!ok)
                atomicExch(&g_stem_tc_error, ESPDL_ERR_TIMEOUT);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..17)
        const int ew = warp - 2;
        const int group = ew >> 2;       // 0..3
        const int acc = group % ST_ACC;  // accumulator buffer this group reads
        const int part = group / ST_ACC; // which half of the tile's 32-column chunks
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
            if (local % ST_ACC != acc)
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
            const int ncols = min(ST_J, p.ow - ST_J * s) * p.cout;
            int8_t *orow = (int8_t *)p.out + (((long long)n * p.oh + y) * p.ow + ST_J * s) * p.cout;
            const uint32_t t0 = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(acc * 256);
            if (fast) {
                // rows are requantised into this group's shared-memory tile and leave through one 3-D TMA store,
                // which also clips the ragged last group of eight outputs and rows outside the image
                const bool leader = (ew & 3) == 0 && lane == 0;
                const uint32_t buf = smem_u32(out_stage + (size_t)group * out_tile_bytes);
                if (leader)
                    bulk_wait_read_all();
                named_bar(2 + group, 128);
                const int col0 = part * out_pw;
                const int floor_q = p.epi.relu ? 0 : INT_MIN;
                if (p.epi.lut)
                    epilogue_stage_lut(t0 + col0, fp + (uint32_t)col0 * 8u, buf, row_in_tile, out_pw, out_pw == 128 ? 7u : 3u, floor_q, smem_u32(lut_s));
                else if (out_pw == 128)
                    epilogue_stage<128>(t0 + col0, fp + (uint32_t)col0 * 8u, buf, row_in_tile, 128, floor_q);
                else
                    epilogue_stage<64>(t0 + col0, fp + (uint32_t)col0 * 8u, buf, row_in_tile, 64, floor_q);
                fence_before();
                fence_async_smem();
                named_bar(2 + group, 128);
                if (leader) {
                    tma_store_3d(&map_out, buf, ST_J * s * p.cout + col0, yb * p.rows_y, ng * p.rows_n);
                    bulk_commit();
                }
            } else {
                int chunk = 0;
                for (int c0 = 0; c0 < ncols; c0 += 16, chunk++) {
                    if ((chunk >> 1) % 2 != part)
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
                    if (row_ok)
                        *(uint4 *)(orow + c0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
            }
            fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(smem_u32(&tempty_bar[acc]));
        }
        if (!ok && lane == 0)
            atomicExch(&g_stem_tc_error, ESPDL_ERR_TIMEOUT);
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

EncodeTiledFn stem_encode()
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

} // namespace

bool conv2d_stem_tc_supported(const espdl_conv_desc &d)
{
    if (d.dtype != ESPDL_DTYPE_INT8 || d.group != 1 || d.kh != 3 || d.kw != 3 || d.in_c != 3)
        return false;
    if (d.stride_h != 2 || d.stride_w != 2 || d.dilation_h != 1 || d.dilation_w != 1)
        return false;
    if (d.pad_top < 0 || d.pad_top > 1 || d.pad_left < 0 || d.pad_left > 1)
        return false;
    if (d.out_c % 16 != 0 || d.out_c > 32) // 8 outputs x Cout columns must fit one accumulator of 256
        return false;
    if ((d.in_pixel_stride && d.in_pixel_stride != 3) || (d.out_pixel_stride && d.out_pixel_stride != d.out_c))
        return false;
    const long long row_bytes = 3ll * d.in_w;
    if (row_bytes % 16 != 0 || ((uintptr_t)d.input % 16) || ((uintptr_t)d.output % 16) || d.in_h < 3)
        return false;
    return true;
}

int conv2d_stem_tc(const espdl_conv_desc &d, cudaStream_t s)
{
    if (!conv2d_stem_tc_supported(d))
        return ESPDL_ERR_UNSUPPORTED;
    EncodeTiledFn enc = stem_encode();
    if (!enc)
        return set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point not found");
    StemParams p;
    p.n = d.n, p.ih = d.in_h, p.iw = d.in_w, p.oh = d.out_h, p.ow = d.out_w, p.cout = d.out_c;
    p.pt = d.pad_top, p.pl = d.pad_left;
    p.rows_n = d.n >= 8 ? 8 : (d.n >= 4 ? 4 : (d.n >= 2 ? 2 : 1));
    p.rows_y = 128 / p.rows_n;
    p.segs = (d.out_w + ST_J - 1) / ST_J;
    p.yblocks = (d.out_h + p.rows_y - 1) / p.rows_y;
    p.ngroups = (d.n + p.rows_n - 1) / p.rows_n;
    p.x_shift = d.pad_left ? 16 : 0;
    p.k_base = d.pad_left ? 16 - 3 * d.pad_left : 0;
    p.w = (const int8_t *)d.filter, p.out = d.output;
    p.epi.bias = d.bias, p.epi.ew = d.filter_exponents, p.epi.lut = d.lut, p.epi.lut_stride = d.lut_channel_stride;
    p.epi.e_shift_base = d.out_exponent - d.in_exponent;
    p.epi.ew_scalar = d.filter_exponent, p.epi.per_channel = d.per_channel;
    p.epi.relu = d.activation == ESPDL_ACT_RELU, p.epi.half_even = d.round_mode == ESPDL_ROUND_HALF_EVEN;

    // One map per filter row ky: input rows 2*y + ky - pad_top = 2*(y + q) + r, so the map starts at row r, steps
    // two rows per index and is addressed with y + q; indices outside [0, rows of that parity) read zeros.
    CUtensorMap maps[3];
    const uint64_t row_bytes = 3ull * d.in_w;
    for (int ky = 0; ky < 3; ky++) {
        const int off = ky - d.pad_top;
        const int r = ((off % 2) + 2) % 2, q = (off - r) / 2;
        p.yq[ky] = q;
        cuuint64_t dims[3] = {row_bytes, (cuuint64_t)((d.in_h - r + 1) / 2), (cuuint64_t)d.n};
        cuuint64_t strides[2] = {2 * row_bytes, (cuuint64_t)d.in_h * row_bytes};
        cuuint32_t box[3] = {ST_K, (cuuint32_t)p.rows_y, (cuuint32_t)p.rows_n};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult res = enc(&maps[ky], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, (void *)((const uint8_t *)d.input + r * row_bytes), dims, strides, box,
                           estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (res != CUDA_SUCCESS)
            return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(stem)");
    }
    // output as a 3-D tensor {OW*Cout bytes, OH, N}; a group's piece is half of a tile row
    CUtensorMap mo;
    {
        const int pw = ST_J * d.out_c / 2;
        cuuint64_t dims[3] = {(cuuint64_t)d.out_w * d.out_c, (cuuint64_t)d.out_h, (cuuint64_t)d.n};
        cuuint64_t strides[2] = {(cuuint64_t)d.out_w * d.out_c, (cuuint64_t)d.out_h * d.out_w * d.out_c};
        cuuint32_t box[3] = {(cuuint32_t)pw, (cuuint32_t)p.rows_y, (cuuint32_t)p.rows_n};
        cuuint32_t estr[3] = {1, 1, 1};
        if (enc(&mo, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, d.output, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                pw == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(stem output)");
    }
    const size_t smem = 1024 + 3 * 256 * ST_K + (size_t)ST_STAGES * 3 * ST_A_BYTES + 4 * 128 * 128 + sizeof(FastParam) * 256 +
        (2 * ST_STAGES + 2 * ST_ACC) * 8 + 32 + 256 + 16;
    static std::once_flag attr_once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(attr_once, [] { attr_err = cudaFuncSetAttribute(stem_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024); });
    if (attr_err != cudaSuccess)
        return set_cuda_error(attr_err, "cudaFuncSetAttribute(stem_tc_kernel)");
    const int total = p.ngroups * p.yblocks * p.segs;
    const int grid = min(total, num_sms());
    stem_tc_kernel<<<grid, ST_THREADS, max(smem, (size_t)120 * 1024), s>>>(maps[0], maps[1], maps[2], mo, p);
    count_launch();
    return check_launch("stem_tc");
}

} // namespace espdl
