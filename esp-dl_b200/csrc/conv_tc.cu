// Dense Conv2D (any filter size, stride 1 or 2, dilation, padding; int8, groups = 1) as an implicit GEMM on the
// tensor cores.  Replaces dl::base::conv2d<int8_t,...> (esp-dl/dl/base/dl_base_conv2d.cpp:9-163, MAC kernels
// conv2d_33cn / conv2d_hwcn) for filters larger than 1x1, with the epilogue of
// esp-dl/dl/base/dl_base_activate_buffer.hpp:27-73.
//
//   out[n, y, x, co] = epilogue( sum_{ky, kx, c} in[n, y*S + ky*D - pt, x*S + kx*D - pl, c] * w[co][ky][kx][c] + bias[co] )
//
// No im2col buffer exists anywhere.  A tile is R rows x P columns of output pixels of one image (R*P <= 128 = the
// M of a tcgen05 MMA) x up to 256 output channels.  The reduction runs over the filter taps: for tap (ky, kx) and a
// block of up to 128 input channels, ONE 4-D TMA box {channels, P, R, 1} of the NHWC input, displaced by the tap
// (and stepping S pixels per index with TMA element strides), lands in shared memory as the K-major swizzled A
// operand whose rows are the tile's pixels; coordinates outside the image are zero-filled by the TMA unit, which is
// the reference's padding rule (taps outside the image contribute nothing).  B is a 2-D box of the [Cout][KH*KW*Cin]
// filter at column (ky*KW + kx)*Cin.  KH*KW*ceil(Cin/128) such stages accumulate into one TMEM accumulator; the
// epilogue is the pointwise tile kernel's (constants of the one-add-one-shift form staged in shared memory, rows
// requantised into a shared tile and moved out by a 4-D TMA store that clips at the image border).
// Roles, barriers and bounded waits are those of gemm_tc.cu.
#include "tc_common.cuh"

#include <mutex>

namespace espdl {

__device__ int g_conv_tc_error = 0;

int read_and_clear_device_error_conv()
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_conv_tc_error, sizeof(int)) != cudaSuccess)
        return 0;
    if (v) {
        int zero = 0;
        cudaMemcpyToSymbol(g_conv_tc_error, &zero, sizeof(int));
    }
    return v;
}

namespace {

using namespace tc;

constexpr int CV_THREADS = 64 + 16 * 32; // TMA warp, MMA warp, 16 epilogue warps in four groups
constexpr int CV_MAX_STAGES = 8;
constexpr int CV_MAX_ACC = 4;
constexpr size_t CV_SMEM_BUDGET = 200 * 1024;

struct ConvTcParams {
    int n, oh, ow, cin, cout;
    int kh, kw, S, D, pt, pl;
    int P, R;                     // tile: R rows x P columns of output pixels
    int xtiles, ytiles, n_tiles;  // tiles per image row / column, tiles along Cout
    int block_n, swz, cblocks;    // Cout per tile, bytes of Cin per stage, stages per tap
    int stages, acc_stages, tmem_cols;
    int out_pw, out_mask;         // staged epilogue: bytes per row of a group's piece (0 = direct row stores), swizzle mask
    void *out;
    long long ops;                // output pixel stride in bytes
    EpiConfig epi;
};

__device__ __forceinline__ void tma_store_4d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2, int c3)
{
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map), "r"(src), "r"(c0), "r"(c1),
                 "r"(c2), "r"(c3)
                 : "memory");
}

__global__ void __launch_bounds__(CV_THREADS, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_out,
               const ConvTcParams p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int a_bytes = 128 * p.swz;
    const int b_bytes = p.block_n * p.swz;
    const int stage_bytes = a_bytes + b_bytes;
    const int n_pad = p.n_tiles * p.block_n;
    uint8_t *out_stage = smem + (size_t)p.stages * stage_bytes;
    const int out_tile_bytes = (128 * p.out_pw + 1023) & ~1023;
    uint8_t *aux = out_stage + 4 * (size_t)out_tile_bytes;
    FastParam *fast_s = (FastParam *)aux;
    uint64_t *bars = (uint64_t *)(aux + sizeof(FastParam) * (size_t)n_pad);
    uint64_t *full_bar = bars, *empty_bar = bars + CV_MAX_STAGES, *tfull_bar = bars + 2 * CV_MAX_STAGES, *tempty_bar = tfull_bar + CV_MAX_ACC;
    uint32_t *tmem_slot = (uint32_t *)(tempty_bar + CV_MAX_ACC);
    int *slow_flag = (int *)(tmem_slot + 1);
    uint8_t *lut_s = (uint8_t *)(slow_flag + 3); // the fused 8-bit table, 256 bytes, 16-byte aligned

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_per_image = p.ytiles * p.xtiles * p.n_tiles;
    const int total_tiles = p.n * tiles_per_image;
    const int parts = 4 / p.acc_stages;
    const int taps = p.kh * p.kw;
    const uint32_t a_tx = (uint32_t)(p.P * p.R * p.swz); // the A box holds P*R rows; rows up to 128 keep stale bytes

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < CV_MAX_ACC; a++) {
            mbar_init(smem_u32(&tfull_bar[a]), 1);
            mbar_init(smem_u32(&tempty_bar[a]), 4 * parts);
        }
        *slow_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1)
        tmem_alloc(smem_u32(tmem_slot), p.tmem_cols);
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
                const int nt = tile % p.n_tiles;
                const int xt = (tile / p.n_tiles) % p.xtiles;
                const int yt = (tile / (p.n_tiles * p.xtiles)) % p.ytiles;
                const int img = tile / tiles_per_image;
                const int n0 = nt * p.block_n;
                for (int tap = 0; tap < taps && ok; tap++) {
                    const int ky = tap / p.kw, kx = tap % p.kw;
                    const int ix = xt * p.P * p.S + kx * p.D - p.pl;
                    const int iy = yt * p.R * p.S + ky * p.D - p.pt;
                    for (int cb = 0; cb < p.cblocks; cb++) {
                        if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1)) {
                            ok = false;
                            break;
                        }
                        const uint32_t bar = smem_u32(&full_bar[stage]);
                        uint8_t *st = smem + (size_t)stage * stage_bytes;
                        mbar_arrive_expect_tx(bar, a_tx + (uint32_t)b_bytes);
                        tma_load_4d(smem_u32(st), &map_a, cb * p.swz, ix, iy, img, bar);
                        tma_load_2d(smem_u32(st + a_bytes), &map_b, tap * p.cin + cb * p.swz, n0, bar);
                        if (++stage == p.stages) {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                }
            }
            if (!ok)
                atomicExch(&g_conv_tc_error, ESPDL_ERR_TIMEOUT);
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            const uint32_t idesc = idesc_i8(1, 1, 128, p.block_n);
            const int ksteps = p.swz / 32;
            const int kblocks = taps * p.cblocks;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1)) {
                    ok = false;
                    break;
                }
                fence_after();
                const uint32_t d0 = tmem_base + (uint32_t)(acc * p.block_n);
                for (int kb = 0; kb < kblocks; kb++) {
                    if (!mbar_wait(smem_u32(&full_bar[stage]), phase)) {
                        ok = false;
                        break;
                    }
                    fence_after();
                    const uint32_t st = smem_u32(smem + (size_t)stage * stage_bytes);
                    const uint64_t da = smem_desc_swizzled(st, p.swz);
                    const uint64_t db = smem_desc_swizzled(st + a_bytes, p.swz);
                    for (int k = 0; k < ksteps; k++) mma_i8(d0, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0);
                    commit(smem_u32(&empty_bar[stage]));
                    if (++stage == p.stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok)
                    break;
                commit(smem_u32(&tfull_bar[acc]));
                if (++acc == p.acc_stages) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
            if (!ok)
                atomicExch(&g_conv_tc_error, ESPDL_ERR_TIMEOUT);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..17)
        const int ew = warp - 2;
        const int group = ew >> 2;
        const int acc = group % p.acc_stages;
        const int part = group / p.acc_stages;
        const int lane_group = warp & 3;
        const int row_in_tile = lane_group * 32 + lane;
        const int et = threadIdx.x - 64;
        stage_fast_params(p.epi, fast_s, p.cout, n_pad, et, 16 * 32, slow_flag);
        if (p.epi.lut)
            stage_lut(p.epi.lut, lut_s, et, 16 * 32);
        asm volatile("bar.sync 1, %0;" ::"n"(16 * 32) : "memory");
        // a fused table rides on the staged form; the direct-store form applies it in its general path
        const bool fast = !*slow_flag && !p.epi.half_even && !p.epi.lut_stride && (long long)p.cin * p.kh * p.kw <= 32768;
        const uint32_t fp_base = epi_param_base(fast_s);
        const int floor_q = p.epi.relu ? 0 : INT_MIN;
        const int ry = row_in_tile / p.P, rx = row_in_tile % p.P;
        uint32_t acc_phase = 0;
        bool ok = true;
        int local = 0;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, local++) {
            if (local % p.acc_stages != acc)
                continue;
            const int nt = tile % p.n_tiles;
            const int xt = (tile / p.n_tiles) % p.xtiles;
            const int yt = (tile / (p.n_tiles * p.xtiles)) % p.ytiles;
            const int img = tile / tiles_per_image;
            const int n0 = nt * p.block_n;
            if (!mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase)) {
                ok = false;
                break;
            }
            acc_phase ^= 1;
            fence_after();
            const uint32_t t0 = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(acc * p.block_n);
            if (fast && p.out_pw) {
                const bool leader = (ew & 3) == 0 && lane == 0;
                const uint32_t buf = smem_u32(out_stage + (size_t)group * out_tile_bytes);
                if (leader)
                    bulk_wait_read_all();
                named_bar(2 + group, 128);
                const int col0 = part * p.out_pw;
                const uint32_t fpp = fp_base + (uint32_t)(n0 + col0) * 8u;
                if (p.epi.lut) {
                    epilogue_stage_lut(t0 + col0, fpp, buf, row_in_tile, p.out_pw, (uint32_t)p.out_mask, floor_q, smem_u32(lut_s));
                } else if (p.out_pw == 128)
                    epilogue_stage<128>(t0 + col0, fpp, buf, row_in_tile, 128, floor_q);
                else if (p.out_pw == 64)
                    epilogue_stage<64>(t0 + col0, fpp, buf, row_in_tile, 64, floor_q);
                else
                    epilogue_stage<0>(t0 + col0, fpp, buf, row_in_tile, p.out_pw, floor_q);
                // the accumulator is free once this warp's TMEM loads are done: hand it back before the tile is stored
                fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(smem_u32(&tempty_bar[acc]));
                fence_async_smem();
                named_bar(2 + group, 128);
                if (leader) {
                    tma_store_4d(&map_out, buf, n0 + col0, xt * p.P, yt * p.R, img); // clipped at the image border and at Cout
                    bulk_commit();
                }
                continue;
            } else {
                // direct rows: any rounding mode, any shift, optional LUT, any alignment
                const int oy = yt * p.R + ry, ox = xt * p.P + rx;
                const bool row_ok = ry < p.R && oy < p.oh && ox < p.ow;
                int8_t *orow = (int8_t *)p.out + (((long long)img * p.oh + oy) * p.ow + ox) * p.ops + n0;
                const uintptr_t amix = (uintptr_t)p.ops | (((uintptr_t)p.out) + (uintptr_t)n0) | 16u;
                const int out_align = (int)(amix & (~amix + 1));
                int chunk = 0;
                for (int c0 = 0; c0 < p.block_n; c0 += 16, chunk++) {
                    if ((chunk >> 1) % parts != part)
                        continue;
                    int32_t v[16];
                    ld16(t0 + c0, v);
                    ld_wait16(v);
                    uint32_t pk[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                    if (fast) {
                        if (p.epi.relu)
                            requant16_fast<true>(v, fast_s + n0 + c0, pk);
                        else
                            requant16_fast<false>(v, fast_s + n0 + c0, pk);
                        if (p.epi.lut) { // a fused table on rows that leave unstaged: same lookups on the packed words
#pragma unroll
                            for (int q = 0; q < 4; q++) pk[q] = lut4(pk[q], smem_u32(lut_s));
                        }
                    } else {
                        requant16_general(v, p.epi, n0 + c0, p.cout, pk);
                    }
                    const int count = min(16, p.cout - (n0 + c0));
                    if (row_ok && count > 0)
                        store_bytes(orow + c0, pk, count, out_align);
                }
            }
            fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(smem_u32(&tempty_bar[acc]));
        }
        if (!ok && lane == 0)
            atomicExch(&g_conv_tc_error, ESPDL_ERR_TIMEOUT);
        if (p.out_pw && (ew & 3) == 0 && lane == 0)
            bulk_wait_all();
    }

    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        tmem_dealloc(tmem_base, p.tmem_cols);
    }
}

// ------------------------------------------------------------------------------------------ stride-1 windows from ONE patch
// The kernel above fetches every input byte once per filter tap (nine boxes of 128 pixels for a 3x3 window), and with
// 32-128 byte rows that traffic, not the MMAs, bounds it (64 -> 64 channels at 80x80: 1.8 GB through the TMA unit for a
// 0.4 GB tensor).  For stride 1, dilation 1 and one channel block the taps are shifted views of the same pixels: here a
// tile's input arrives as ONE 4-D box {Cin, PW pixels, RT + KH - 1 rows, 1 image} whose dense shared-memory image is
// a run of "flat positions" row * PW + x, and tap (ky, kx) is the same run started (ky * PW + kx) rows later - a
// descriptor start address, no data movement (the swizzle is a function of the absolute shared-memory address, so a
// start moved by whole rows stays consistent with what the TMA unit wrote).  The 128 rows of an MMA are 128 consecutive
// flat positions = RT = 128 / PW image rows of PW positions, of which the last KW - 1 of every row are not outputs (their
// windows run into the next row); they are computed and dropped.  The whole filter stays in shared memory for the life of
// the CTA.  Borders are TMA zero fill.  Epilogue and roles as above; a tile leaves through one TMA store per image row.
struct PatchParams {
    int n, oh, ow, cin, cout;
    int kh, kw, pt, pl;
    int PW, RT, PV;               // positions per patch row (32, 64 or 128), image rows per tile, outputs per row = PW - (KW - 1)
    int xtiles, ytiles;
    int block_n, swz;
    int stages, acc_stages, tmem_cols;
    int patch_bytes, patch_tx;    // shared-memory stride of a stage (with slack for the last taps' overrun), bytes one box delivers
    int out_pw, out_mask;
    int stack, ncols;             // the first `stack` taps of a filter row side by side along N (0: none); ncols = accumulator columns per tile
    int staged;                   // the tile leaves through shared memory and TMA stores (else rows go out of registers)
    void *out;
    long long ops;                // output pixel stride in bytes
    EpiConfig epi;
};

// Stacked taps: accumulator column block kx of TMEM lane m holds tap column kx's share of the output at position m - kx,
// so an output is the sum over kx of block kx read kx lanes further on.  With 32 positions per patch row a warp's 32
// lanes are exactly one image row and the last KW - 1 of them are dropped, so the shuffles never leave the warp.
__device__ __forceinline__ void ld16_sum(uint32_t t, int kw, int stride, int32_t *v)
{
    ld16(t, v);
    ld_wait16(v);
    for (int kx = 1; kx < kw; kx++) {
        int32_t u[16];
        ld16(t + (uint32_t)(kx * stride), u);
        ld_wait16(u);
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] += __shfl_down_sync(0xffffffffu, u[i], kx);
    }
}

static __device__ __noinline__ void epilogue_stage_stacked(uint32_t t0, int kw, int stride, uint32_t fp, uint32_t buf, int row, int pw, uint32_t mask,
                                                           int floor_q, uint32_t tbl)
{
    const uint32_t rx = ((((uint32_t)(row * pw)) >> 7) & mask) << 4;
    const uint32_t rb = buf + (uint32_t)(row * pw);
    if (kw == 3) {
        // three column blocks per chunk, the next chunk's loads in flight while this one is requantised
        int32_t a0[16], a1[16], a2[16];
        ld16(t0, a0);
        ld16(t0 + (uint32_t)stride, a1);
        ld16(t0 + (uint32_t)(2 * stride), a2);
#pragma unroll 1
        for (int c = 0; c < pw; c += 16) {
            int32_t v[16];
            uint32_t pk[4];
            ld_wait16(a0);
            tie16(a1);
            tie16(a2);
#pragma unroll
            for (int i = 0; i < 16; i++) v[i] = a0[i] + __shfl_down_sync(0xffffffffu, a1[i] + __shfl_down_sync(0xffffffffu, a2[i], 1), 1);
            tie16(v);
            if (c + 16 < pw) {
                ld16(t0 + (uint32_t)(c + 16), a0);
                ld16(t0 + (uint32_t)(c + 16 + stride), a1);
                ld16(t0 + (uint32_t)(c + 16 + 2 * stride), a2);
            }
#pragma unroll
            for (int q = 0; q < 4; q++) {
                pk[q] = requant4_floor(v + 4 * q, fp + (uint32_t)(c + 4 * q) * 8u, floor_q);
                if (tbl)
                    pk[q] = lut4(pk[q], tbl);
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rb + ((uint32_t)c ^ rx)), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3])
                         : "memory");
        }
        return;
    }
#pragma unroll 1
    for (int c = 0; c < pw; c += 16) {
        int32_t v[16];
        uint32_t pk[4];
        ld16_sum(t0 + c, kw, stride, v);
#pragma unroll
        for (int q = 0; q < 4; q++) {
            pk[q] = requant4_floor(v + 4 * q, fp + (uint32_t)(c + 4 * q) * 8u, floor_q);
            if (tbl)
                pk[q] = lut4(pk[q], tbl);
        }
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rb + ((uint32_t)c ^ rx)), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3])
                     : "memory");
    }
}

__global__ void __launch_bounds__(CV_THREADS, 1)
conv_patch_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_out,
                  const __grid_constant__ PatchParams p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int taps = p.kh * p.kw;
    const int b_tap = p.block_n * p.swz;                       // one tap's filter rows: whole swizzle patterns (block_n % 16 == 0)
    uint8_t *filt_s = smem;                                    // taps x [block_n][swz]
    uint8_t *patch_s = smem + (size_t)taps * b_tap;            // stages x patch
    uint8_t *out_stage = patch_s + (size_t)p.stages * p.patch_bytes;
    const int out_tile_bytes = p.staged ? (128 * p.out_pw + 1023) & ~1023 : 0;
    uint8_t *aux = out_stage + 4 * (size_t)out_tile_bytes;
    FastParam *fast_s = (FastParam *)aux;
    uint64_t *bars = (uint64_t *)(aux + sizeof(FastParam) * (size_t)p.block_n);
    uint64_t *full_bar = bars, *empty_bar = bars + CV_MAX_STAGES, *tfull_bar = bars + 2 * CV_MAX_STAGES, *tempty_bar = tfull_bar + CV_MAX_ACC;
    uint64_t *filt_bar = tempty_bar + CV_MAX_ACC;
    uint32_t *tmem_slot = (uint32_t *)(filt_bar + 1);
    int *slow_flag = (int *)(tmem_slot + 1);
    uint8_t *lut_s = (uint8_t *)(slow_flag + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_per_image = p.ytiles * p.xtiles;
    const int total_tiles = p.n * tiles_per_image;
    const int parts = 4 / p.acc_stages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < CV_MAX_ACC; a++) {
            mbar_init(smem_u32(&tfull_bar[a]), 1);
            mbar_init(smem_u32(&tempty_bar[a]), 4 * parts);
        }
        mbar_init(smem_u32(filt_bar), 1);
        *slow_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1)
        tmem_alloc(smem_u32(tmem_slot), p.tmem_cols);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // the filter, once: one box per tap
            mbar_arrive_expect_tx(smem_u32(filt_bar), (uint32_t)(taps * b_tap));
            for (int tap = 0; tap < taps; tap++) tma_load_2d(smem_u32(filt_s + (size_t)tap * b_tap), &map_b, tap * p.cin, 0, smem_u32(filt_bar));
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int xt = tile % p.xtiles;
                const int yt = (tile / p.xtiles) % p.ytiles;
                const int img = tile / tiles_per_image;
                if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1)) {
                    ok = false;
                    break;
                }
                const uint32_t bar = smem_u32(&full_bar[stage]);
                mbar_arrive_expect_tx(bar, (uint32_t)p.patch_tx);
                tma_load_4d(smem_u32(patch_s + (size_t)stage * p.patch_bytes), &map_a, 0, xt * p.PV - p.pl, yt * p.RT - p.pt, img, bar);
                if (++stage == p.stages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (!ok)
                atomicExch(&g_conv_tc_error, ESPDL_ERR_TIMEOUT);
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = mbar_wait(smem_u32(filt_bar), 0);
            const uint32_t idesc = idesc_i8(1, 1, 128, p.ncols), idesc_one = idesc_i8(1, 1, 128, p.block_n);
            const int ksteps = p.swz / 32;
            const uint32_t f0 = smem_u32(filt_s);
            const int wide = p.stack ? p.stack : 1;    // taps the first MMA of a filter row covers; the others follow one by one
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1) || !mbar_wait(smem_u32(&full_bar[stage]), phase)) {
                    ok = false;
                    break;
                }
                fence_after();
                const uint32_t d0 = tmem_base + (uint32_t)(acc * p.ncols);
                const uint32_t st = smem_u32(patch_s + (size_t)stage * p.patch_bytes);
                int first = 1;
                for (int ky = 0; ky < p.kh; ky++)
                    for (int kx = 0; kx < p.kw; kx += (kx == 0 ? wide : 1)) {
                        // a single tap behind the stacked ones adds to column block 0 from rows kx further on
                        const uint64_t da = smem_desc_swizzled(st + (uint32_t)((ky * p.PW + kx) * p.swz), p.swz);
                        const uint64_t db = smem_desc_swizzled(f0 + (uint32_t)((ky * p.kw + kx) * b_tap), p.swz);
                        const uint32_t id = kx == 0 ? idesc : idesc_one;
                        for (int k = 0; k < ksteps; k++, first = 0) mma_i8(d0, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), id, !first);
                    }
                commit(smem_u32(&empty_bar[stage]));
                commit(smem_u32(&tfull_bar[acc]));
                if (++stage == p.stages) {
                    stage = 0;
                    phase ^= 1;
                }
                if (++acc == p.acc_stages) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
            if (!ok)
                atomicExch(&g_conv_tc_error, ESPDL_ERR_TIMEOUT);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..17)
        const int ew = warp - 2;
        const int group = ew >> 2;
        const int acc = group % p.acc_stages;
        const int part = group / p.acc_stages;
        const int lane_group = warp & 3;
        const int row_in_tile = lane_group * 32 + lane;
        const int et = threadIdx.x - 64;
        stage_fast_params(p.epi, fast_s, p.cout, p.block_n, et, 16 * 32, slow_flag);
        if (p.epi.lut)
            stage_lut(p.epi.lut, lut_s, et, 16 * 32);
        asm volatile("bar.sync 1, %0;" ::"n"(16 * 32) : "memory");
        const bool fast = !*slow_flag && !p.epi.half_even && !p.epi.lut_stride && (long long)p.cin * p.kh * p.kw <= 32768;
        const uint32_t fp_base = epi_param_base(fast_s);
        const int floor_q = p.epi.relu ? 0 : INT_MIN;
        uint32_t acc_phase = 0;
        bool ok = true;
        int local = 0;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, local++) {
            if (local % p.acc_stages != acc)
                continue;
            const int xt = tile % p.xtiles;
            const int yt = (tile / p.xtiles) % p.ytiles;
            const int img = tile / tiles_per_image;
            if (!mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase)) {
                ok = false;
                break;
            }
            acc_phase ^= 1;
            fence_after();
            const uint32_t t0 = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(acc * p.ncols);
            if (!fast) {
                // direct rows: any rounding mode, any shift, optional table
                const int r = row_in_tile / p.PW, xx = row_in_tile % p.PW;
                const int oy = yt * p.RT + r, ox = xt * p.PV + xx;
                const bool row_ok = xx < p.PV && oy < p.oh && ox < p.ow;
                int8_t *orow = (int8_t *)p.out + (((long long)img * p.oh + oy) * p.ow + ox) * p.ops;
                const uintptr_t amix = (uintptr_t)p.ops | ((uintptr_t)p.out) | 16u;
                const int out_align = (int)(amix & (~amix + 1));
                for (int c0 = part * p.out_pw; c0 < (part + 1) * p.out_pw; c0 += 16) {
                    int32_t v[16];
                    ld16_sum(t0 + c0, p.stack ? p.stack : 1, p.block_n, v);
                    uint32_t pk[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                    requant16_general(v, p.epi, c0, p.cout, pk);
                    const int count = min(16, p.cout - c0);
                    if (row_ok && count > 0)
                        store_bytes(orow + c0, pk, count, out_align);
                }
                fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(smem_u32(&tempty_bar[acc]));
                continue;
            }
            const int col0 = part * p.out_pw;
            const uint32_t fpp = fp_base + (uint32_t)col0 * 8u;
            if (!p.staged) {
                // no room for staging tiles next to a large resident filter: 16 bytes of the thread's own row per store
                const int r = row_in_tile / p.PW, xx = row_in_tile % p.PW;
                const int oy = yt * p.RT + r, ox = xt * p.PV + xx;
                const bool row_ok = xx < p.PV && oy < p.oh && ox < p.ow;
                int8_t *orow = (int8_t *)p.out + (((long long)img * p.oh + oy) * p.ow + ox) * p.ops + col0;
                const uint32_t tbl = p.epi.lut ? smem_u32(lut_s) : 0u;
                for (int c = 0; c < p.out_pw; c += 16) {
                    int32_t v[16];
                    uint32_t pk[4];
                    ld16_sum(t0 + col0 + c, p.stack ? p.stack : 1, p.block_n, v);
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        pk[q] = requant4_floor(v + 4 * q, fpp + (uint32_t)(c + 4 * q) * 8u, floor_q);
                        if (tbl)
                            pk[q] = lut4(pk[q], tbl);
                    }
                    if (row_ok)
                        *(uint4 *)(orow + c) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
                fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(smem_u32(&tempty_bar[acc]));
                continue;
            }
            const bool leader = (ew & 3) == 0 && lane == 0;
            const uint32_t buf = smem_u32(out_stage + (size_t)group * out_tile_bytes);
            if (leader)
                bulk_wait_read_all();
            named_bar(2 + group, 128);
            if (p.stack)
                epilogue_stage_stacked(t0 + col0, p.stack, p.block_n, fpp, buf, row_in_tile, p.out_pw, (uint32_t)p.out_mask, floor_q,
                                       p.epi.lut ? smem_u32(lut_s) : 0u);
            else if (p.epi.lut)
                epilogue_stage_lut(t0 + col0, fpp, buf, row_in_tile, p.out_pw, (uint32_t)p.out_mask, floor_q, smem_u32(lut_s));
            else if (p.out_pw == 128)
                epilogue_stage<128>(t0 + col0, fpp, buf, row_in_tile, 128, floor_q);
            else if (p.out_pw == 64)
                epilogue_stage<64>(t0 + col0, fpp, buf, row_in_tile, 64, floor_q);
            else
                epilogue_stage<0>(t0 + col0, fpp, buf, row_in_tile, p.out_pw, floor_q);
            fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(smem_u32(&tempty_bar[acc]));
            fence_async_smem();
            named_bar(2 + group, 128);
            if (leader) {
                // one store per image row of the tile: PV outputs of out_pw channels; rows and columns outside the image are clipped
                for (int r = 0; r < p.RT; r++) tma_store_4d(&map_out, buf + (uint32_t)(r * p.PW * p.out_pw), col0, xt * p.PV, yt * p.RT + r, img);
                bulk_commit();
            }
        }
        if (!ok && lane == 0)
            atomicExch(&g_conv_tc_error, ESPDL_ERR_TIMEOUT);
        if ((ew & 3) == 0 && lane == 0)
            bulk_wait_all();
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

EncodeTiledFn conv_encode()
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

CUtensorMapSwizzle swizzle_of(int bytes)
{
    return bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
        : (bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : (bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE));
}

size_t conv_aux_bytes(const ConvTcParams &p) { return sizeof(FastParam) * (size_t)p.n_tiles * p.block_n + (2 * CV_MAX_STAGES + 2 * CV_MAX_ACC) * 8 + 32 + 256; }

bool conv_plan(const espdl_conv_desc &d, ConvTcParams &p)
{
    p.n = d.n, p.oh = d.out_h, p.ow = d.out_w, p.cin = d.in_c, p.cout = d.out_c;
    p.kh = d.kh, p.kw = d.kw, p.S = d.stride_h, p.D = d.dilation_h, p.pt = d.pad_top, p.pl = d.pad_left;
    // tile shape: the R x P (R*P <= 128) that wastes the fewest accumulator rows on this image
    double best = -1;
    p.P = 1, p.R = 1;
    for (int P = 1; P <= 128 && P <= d.out_w && P * p.S <= 256; P++) {
        const int R = min(128 / P, min(d.out_h, 256 / p.S));
        if (R < 1)
            continue;
        const double eff = ((double)d.out_w / (((d.out_w + P - 1) / P) * P)) * ((double)d.out_h / (((d.out_h + R - 1) / R) * R)) * (P * R / 128.0);
        if (eff > best + 1e-9) {
            best = eff;
            p.P = P, p.R = R;
        }
    }
    p.xtiles = (d.out_w + p.P - 1) / p.P, p.ytiles = (d.out_h + p.R - 1) / p.R;
    p.n_tiles = (p.cout + 255) / 256;
    p.block_n = (((p.cout + p.n_tiles - 1) / p.n_tiles) + 15) / 16 * 16;
    if (p.block_n > 128)
        p.block_n = (p.block_n + 31) / 32 * 32;
    p.n_tiles = (p.cout + p.block_n - 1) / p.block_n;
    p.swz = p.cin >= 96 ? 128 : (p.cin > 32 ? 64 : 32);
    p.cblocks = (p.cin + p.swz - 1) / p.swz;
    p.acc_stages = 4 * p.block_n <= 512 ? 4 : 2;
    int pow2 = 32;
    while (pow2 < p.acc_stages * p.block_n) pow2 *= 2;
    if (pow2 > 512)
        return false;
    p.tmem_cols = pow2;
    const long long ops = d.out_pixel_stride ? d.out_pixel_stride : d.out_c;
    p.out_pw = 0, p.out_mask = 0;
    if (ops % 16 == 0 && ((uintptr_t)d.output % 16) == 0 && !getenv("ESPDL_B200_DIRECT_STORES")) {
        const int parts = 4 / p.acc_stages;
        if (p.block_n % (16 * parts) == 0 && p.block_n / parts <= 128) {
            p.out_pw = p.block_n / parts;
            p.out_mask = p.out_pw == 128 ? 7 : (p.out_pw == 64 ? 3 : 0);
        }
    }
    const size_t stage_bytes = (size_t)(128 + p.block_n) * p.swz;
    size_t out_bytes = 4 * (size_t)((128 * p.out_pw + 1023) & ~1023);
    long long stages = ((long long)CV_SMEM_BUDGET - (long long)conv_aux_bytes(p) - (long long)out_bytes - 1024) / (long long)stage_bytes;
    if (p.out_pw && stages < 4) { // a long reduction needs the deep load pipeline more than the output needs staging
        p.out_pw = 0, p.out_mask = 0, out_bytes = 0;
        stages = ((long long)CV_SMEM_BUDGET - (long long)conv_aux_bytes(p) - 1024) / (long long)stage_bytes;
    }
    if (stages < 2)
        return false;
    p.stages = stages > CV_MAX_STAGES ? CV_MAX_STAGES : (int)stages;
    return true;
}

// The one-patch kernel may use all of an SM's shared memory (227 KB per CTA): a resident 3x3 filter over 128 -> 128
// channels is 144 KB, and what is left decides between two and three patches in flight.
constexpr size_t PATCH_SMEM_BUDGET = 226 * 1024;

size_t patch_aux_bytes(const PatchParams &p) { return sizeof(FastParam) * (size_t)p.block_n + (2 * CV_MAX_STAGES + 2 * CV_MAX_ACC + 1) * 8 + 32 + 256; }

// The one-patch form: stride 1, dilation 1, Cin = 64 or 128 (one swizzle row per pixel), Cout <= 256 in one tile, the
// filter small enough to stay in shared memory next to two or more patches, and the staged epilogue's alignment.
bool patch_plan(const espdl_conv_desc &d, PatchParams &p)
{
    if (getenv("ESPDL_B200_NO_CONV_PATCH"))
        return false;
    if (d.stride_h != 1 || d.stride_w != 1 || d.dilation_h != 1 || d.dilation_w != 1 || (d.in_c != 32 && d.in_c != 64 && d.in_c != 128))
        return false;
    if (d.out_c > 256 || d.out_c % 16 != 0 || d.kw > 8 || d.kh > 8 || d.kh * d.kw < 2)
        return false;
    const long long ops = d.out_pixel_stride ? d.out_pixel_stride : d.out_c;
    if (ops % 16 != 0 || ((uintptr_t)d.output % 16) != 0)
        return false;
    p.n = d.n, p.oh = d.out_h, p.ow = d.out_w, p.cin = d.in_c, p.cout = d.out_c;
    p.kh = d.kh, p.kw = d.kw, p.pt = d.pad_top, p.pl = d.pad_left;
    p.swz = d.in_c, p.block_n = d.out_c;
    // An MMA of 128 rows costs the tensor pipe about the same time for any N up to 256, so as many taps of a filter row
    // as fit into 256 columns (at most four) go side by side along N, if the epilogue's channel split stays a multiple of 16.
    // Filter rows wider than that keep their first taps stacked and issue the others one by one into column block 0.
    p.stack = 0, p.ncols = p.block_n;
    const int fit = std::min(std::min(d.kw, 256 / p.block_n), 4);
    if (fit >= 2 && !getenv("ESPDL_B200_NO_TAP_STACK")) {
        const int acc = 4 * fit * p.block_n <= 512 ? 4 : 2;
        if (p.block_n % (16 * (4 / acc)) == 0)
            p.stack = fit, p.ncols = fit * p.block_n;
    }
    p.acc_stages = 4 * p.ncols <= 512 ? 4 : 2;
    int pow2 = 32;
    while (pow2 < p.acc_stages * p.ncols) pow2 *= 2;
    p.tmem_cols = pow2;
    const int parts = 4 / p.acc_stages;
    if (p.block_n % (16 * parts) != 0 || p.block_n / parts > 128)
        return false;
    p.out_pw = p.block_n / parts;
    p.out_mask = p.out_pw == 128 ? 7 : (p.out_pw == 64 ? 3 : 0);
    // positions per patch row: the width that wastes the fewest of an MMA's 128 rows on this image (stacked taps: 32,
    // one warp of the epilogue per image row)
    double best = -1;
    p.PW = 0;
    for (int PW : {32, 64, 128}) {
        const int PV = PW - (d.kw - 1), RT = 128 / PW;
        if (PV < 8 || (p.stack && PW != 32))
            continue;
        const int xt = (d.out_w + PV - 1) / PV, yt = (d.out_h + RT - 1) / RT;
        const double eff = (double)d.out_w * d.out_h / ((double)xt * PW * yt * RT);
        if (eff > best + 1e-9)
            best = eff, p.PW = PW;
    }
    if (!p.PW)
        return false;
    p.RT = 128 / p.PW, p.PV = p.PW - (d.kw - 1);
    p.xtiles = (d.out_w + p.PV - 1) / p.PV, p.ytiles = (d.out_h + p.RT - 1) / p.RT;
    const int rows = (p.RT + d.kh - 1) * p.PW;
    p.patch_tx = rows * p.swz;
    p.patch_bytes = ((rows + d.kw) * p.swz + 1023) & ~1023; // the last taps of the last (dropped) positions read a few rows further
    const size_t filt = (size_t)d.kh * d.kw * p.block_n * p.swz;
    const size_t out_bytes = 4 * (size_t)((128 * p.out_pw + 1023) & ~1023);
    const long long room = (long long)PATCH_SMEM_BUDGET - (long long)filt - (long long)patch_aux_bytes(p) - 1024;
    p.staged = 1;
    long long stages = (room - (long long)out_bytes) / p.patch_bytes;
    if (stages < 2) { // a filter that leaves no room for the staging tiles: rows go out of registers (long reductions, the epilogue is a small part)
        p.staged = 0;
        stages = room / p.patch_bytes;
    }
    if (stages < 2)
        return false;
    p.stages = stages > 4 ? 4 : (int)stages;
    return true;
}

int launch_patch(const espdl_conv_desc &d, PatchParams &p, cudaStream_t s)
{
    EncodeTiledFn enc = conv_encode();
    if (!enc)
        return set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point not found");
    const int ips = d.in_pixel_stride ? d.in_pixel_stride : d.in_c;
    p.out = d.output;
    p.ops = d.out_pixel_stride ? d.out_pixel_stride : d.out_c;
    p.epi.bias = d.bias, p.epi.ew = d.filter_exponents, p.epi.lut = d.lut, p.epi.lut_stride = d.lut_channel_stride;
    p.epi.e_shift_base = d.out_exponent - d.in_exponent;
    p.epi.ew_scalar = d.filter_exponent, p.epi.per_channel = d.per_channel;
    p.epi.relu = d.activation == ESPDL_ACT_RELU, p.epi.half_even = d.round_mode == ESPDL_ROUND_HALF_EVEN;
    CUtensorMap ma, mb, mo;
    {
        cuuint64_t dims[4] = {(cuuint64_t)d.in_c, (cuuint64_t)d.in_w, (cuuint64_t)d.in_h, (cuuint64_t)d.n};
        cuuint64_t strides[3] = {(cuuint64_t)ips, (cuuint64_t)ips * d.in_w, (cuuint64_t)ips * d.in_w * d.in_h};
        cuuint32_t box[4] = {(cuuint32_t)p.swz, (cuuint32_t)p.PW, (cuuint32_t)(p.RT + d.kh - 1), 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        if (enc(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(d.input), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                swizzle_of(p.swz), CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(conv patch input)");
    }
    {
        const cuuint64_t krow = (cuuint64_t)d.kh * d.kw * d.in_c;
        cuuint64_t dims[2] = {krow, (cuuint64_t)d.out_c};
        cuuint64_t strides[1] = {krow};
        cuuint32_t box[2] = {(cuuint32_t)p.swz, (cuuint32_t)p.block_n};
        cuuint32_t estr[2] = {1, 1};
        if (enc(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(d.filter), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                swizzle_of(p.swz), CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(conv patch filter)");
    }
    {
        cuuint64_t dims[4] = {(cuuint64_t)d.out_c, (cuuint64_t)d.out_w, (cuuint64_t)d.out_h, (cuuint64_t)d.n};
        cuuint64_t strides[3] = {(cuuint64_t)p.ops, (cuuint64_t)p.ops * d.out_w, (cuuint64_t)p.ops * d.out_w * d.out_h};
        cuuint32_t box[4] = {(cuuint32_t)p.out_pw, (cuuint32_t)p.PV, 1, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        if (enc(&mo, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, d.output, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                swizzle_of(p.out_pw == 128 ? 128 : (p.out_pw == 64 ? 64 : 0)), CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(conv patch output)");
    }
    size_t smem = 1024 + (size_t)d.kh * d.kw * p.block_n * p.swz + (size_t)p.stages * p.patch_bytes +
        (p.staged ? 4 * (size_t)((128 * p.out_pw + 1023) & ~1023) : 0) + patch_aux_bytes(p);
    if (smem < 120 * 1024)
        smem = 120 * 1024;
    static std::once_flag attr_once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(attr_once, [] { attr_err = cudaFuncSetAttribute(conv_patch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(PATCH_SMEM_BUDGET + 1024)); });
    if (attr_err != cudaSuccess)
        return set_cuda_error(attr_err, "cudaFuncSetAttribute(conv_patch_kernel)");
    const long long total = (long long)p.n * p.ytiles * p.xtiles;
    if (total > 0x7fffffffll)
        return ESPDL_ERR_TOO_LARGE;
    conv_patch_kernel<<<(int)min(total, (long long)num_sms()), CV_THREADS, smem, s>>>(ma, mb, mo, p);
    count_launch();
    return check_launch("conv_patch");
}

} // namespace

bool conv2d_conv_tc_supported(const espdl_conv_desc &d)
{
    if (d.dtype != ESPDL_DTYPE_INT8 || d.group != 1 || d.n <= 0)
        return false;
    if (d.kh < 1 || d.kw < 1 || d.kh * d.kw > 49 || (d.kh == 1 && d.kw == 1 && d.stride_h == 1))
        return false; // 1x1 stride 1 is the pointwise tile kernel's
    if (d.stride_h != d.stride_w || (d.stride_h != 1 && d.stride_h != 2) || d.dilation_h != d.dilation_w || d.dilation_h < 1 || d.dilation_h > 8)
        return false;
    const int ips = d.in_pixel_stride ? d.in_pixel_stride : d.in_c;
    if (d.in_c % 16 || ips % 16 || ((uintptr_t)d.input % 16) || ((uintptr_t)d.filter % 16) || d.out_c > 8192)
        return false;
    if (d.pad_top < 0 || d.pad_left < 0 || d.in_w > (1 << 20) || d.in_h > (1 << 20))
        return false;
    ConvTcParams p;
    return conv_plan(d, p);
}

int conv2d_conv_tc(const espdl_conv_desc &d, cudaStream_t s)
{
    ConvTcParams p;
    if (!conv2d_conv_tc_supported(d) || !conv_plan(d, p))
        return ESPDL_ERR_UNSUPPORTED;
    {
        PatchParams pp;
        memset(&pp, 0, sizeof(pp));
        if (patch_plan(d, pp))
            return launch_patch(d, pp, s);
    }
    EncodeTiledFn enc = conv_encode();
    if (!enc)
        return set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point not found");
    const int ips = d.in_pixel_stride ? d.in_pixel_stride : d.in_c;
    p.out = d.output;
    p.ops = d.out_pixel_stride ? d.out_pixel_stride : d.out_c;
    p.epi.bias = d.bias, p.epi.ew = d.filter_exponents, p.epi.lut = d.lut, p.epi.lut_stride = d.lut_channel_stride;
    p.epi.e_shift_base = d.out_exponent - d.in_exponent;
    p.epi.ew_scalar = d.filter_exponent, p.epi.per_channel = d.per_channel;
    p.epi.relu = d.activation == ESPDL_ACT_RELU, p.epi.half_even = d.round_mode == ESPDL_ROUND_HALF_EVEN;

    CUtensorMap ma, mb, mo;
    {
        cuuint64_t dims[4] = {(cuuint64_t)d.in_c, (cuuint64_t)d.in_w, (cuuint64_t)d.in_h, (cuuint64_t)d.n};
        cuuint64_t strides[3] = {(cuuint64_t)ips, (cuuint64_t)ips * d.in_w, (cuuint64_t)ips * d.in_w * d.in_h};
        cuuint32_t box[4] = {(cuuint32_t)p.swz, (cuuint32_t)(p.P * p.S), (cuuint32_t)(p.R * p.S), 1};
        cuuint32_t estr[4] = {1, (cuuint32_t)p.S, (cuuint32_t)p.S, 1};
        if (enc(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(d.input), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                swizzle_of(p.swz), CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(conv input)");
    }
    {
        const cuuint64_t krow = (cuuint64_t)d.kh * d.kw * d.in_c;
        cuuint64_t dims[2] = {krow, (cuuint64_t)d.out_c};
        cuuint64_t strides[1] = {krow};
        cuuint32_t box[2] = {(cuuint32_t)p.swz, (cuuint32_t)p.block_n};
        cuuint32_t estr[2] = {1, 1};
        if (enc(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(d.filter), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                swizzle_of(p.swz), CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(conv filter)");
    }
    mo = ma;
    if (p.out_pw) {
        cuuint64_t dims[4] = {(cuuint64_t)d.out_c, (cuuint64_t)d.out_w, (cuuint64_t)d.out_h, (cuuint64_t)d.n};
        cuuint64_t strides[3] = {(cuuint64_t)p.ops, (cuuint64_t)p.ops * d.out_w, (cuuint64_t)p.ops * d.out_w * d.out_h};
        cuuint32_t box[4] = {(cuuint32_t)p.out_pw, (cuuint32_t)p.P, (cuuint32_t)p.R, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        if (enc(&mo, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, d.output, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                swizzle_of(p.out_pw == 128 ? 128 : (p.out_pw == 64 ? 64 : 0)), CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(conv output)");
    }
    const size_t stage_bytes = (size_t)(128 + p.block_n) * p.swz;
    size_t smem = 1024 + (size_t)p.stages * stage_bytes + 4 * (size_t)((128 * p.out_pw + 1023) & ~1023) + conv_aux_bytes(p);
    if (smem < 120 * 1024)
        smem = 120 * 1024; // one CTA per SM, so that TMEM allocation never waits on a neighbour
    static std::once_flag attr_once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(attr_once, [] { attr_err = cudaFuncSetAttribute(conv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(CV_SMEM_BUDGET + 2048)); });
    if (attr_err != cudaSuccess)
        return set_cuda_error(attr_err, "cudaFuncSetAttribute(conv_tc_kernel)");
    const long long total = (long long)p.n * p.ytiles * p.xtiles * p.n_tiles;
    if (total > 0x7fffffffll)
        return ESPDL_ERR_TOO_LARGE;
    const int grid = (int)min(total, (long long)num_sms());
    conv_tc_kernel<<<grid, CV_THREADS, smem, s>>>(ma, mb, mo, p);
    count_launch();
    return check_launch("conv_tc");
}

} // namespace espdl
