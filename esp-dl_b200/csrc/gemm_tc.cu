// Tensor-core (tcgen05) tile kernel for pointwise Conv2D / Gemm / MatMul, int8 and int16.
//
//   out[m, n] = epilogue( sum_k A[m, k] * W[n][k] + bias[n] )         m = pixel, n = output channel
//
// Replaces dl::base::conv2d<> for 1x1 filters (esp-dl/dl/base/dl_base_conv2d.cpp:9-60 conv2d_11cn,
// epilogue esp-dl/dl/base/dl_base_activate_buffer.hpp:27-73), which is also what Gemm and MatMul
// run (esp-dl/dl/module/include/dl_module_gemm.hpp:85-123).
//
// Structure (one persistent CTA per SM, 18 warps):
//   warp 0    TMA producer: cp.async.bulk.tensor 2-D tiles of A (128 rows x SWZ bytes of K) and of W (BLOCK_N rows x
//             SWZ bytes) into a ring of shared-memory stages, swizzled so that the MMA reads them without bank
//             conflicts; rows/columns past the tensor are zero-filled by the TMA unit, so ragged M, N and K need no
//             separate code.
//   warp 1    MMA issuer: one thread issues tcgen05.mma kind::i8 (M=128, N=BLOCK_N, K=32 per instruction), accumulating
//             int32 in TMEM; tcgen05.commit releases the stage and, at the end of a tile, hands the accumulator over.
//   warps 2-17 epilogue, four groups of four warps (a warp may read only its quarter of the 128 TMEM lanes).  With
//             four accumulator buffers each group owns one buffer and every fourth tile; with two buffers two groups
//             share a tile and split its columns.  Each thread owns one output row: tcgen05.ld, bias + ESP-DL's
//             shift/round/saturate with per-channel shifts, ReLU, optional 8-bit LUT, 256-bit NHWC stores.
//             Most layers the network workloads bring are memory bound with a few hundred int8 outputs per input
//             row, so the epilogue's instruction count per output decides the kernel's speed: per-channel constants
//             are staged once in shared memory in a form that needs one add and one shift per output (see
//             tc_common.cuh), and saturation happens inside the pack instruction.
//
// int16 operands: Blackwell tensor cores have no 16-bit integer MMA.  Each operand is split into a signed high byte
// and an unsigned low byte (x = 256*hi + lo); a pre-pass writes the byte planes to scratch, and the tile kernel
// accumulates hi*hi, hi*lo + lo*hi and lo*lo in three TMEM accumulators (kind::i8 takes signedness per operand),
// recombined in 64 bits by the epilogue.  Exact as long as K <= 16384 (the partial sums stay below 2^31).
//
// Every mbarrier wait is bounded (about two seconds); on expiry the kernel records ESPDL_ERR_TIMEOUT in a device word
// that espdl_b200_stream_sync reports, and all roles leave.
#include "tc_common.cuh"

#include <mutex>

namespace espdl {

__device__ int g_tc_error = 0;

int read_and_clear_device_error()
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)) != cudaSuccess)
        return 0;
    if (v) {
        int zero = 0;
        cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
    }
    return v;
}

// Role cycle counters of the tile kernel, compiled in only with -DESPDL_TC_TIMING (a measurement build; the product
// build carries none of it): per CTA, cycles the producer waited for a free stage, the MMA issuer waited for an
// accumulator / for a stage / spent issuing, and epilogue group 0 waited for an accumulator / spent working.
#ifdef ESPDL_TC_TIMING
__device__ long long g_tc_timing[256 * 8];
#define TC_LAP_INIT long long t_ = clock64()
#define TC_LAP(var) do { const long long n_ = clock64(); (var) += n_ - t_; t_ = n_; } while (0)
#define TC_REC(slot, var) g_tc_timing[blockIdx.x * 8 + (slot)] = (var)
__device__ long long g_tc_clock[256 * 4]; // per CTA: clock64 and globaltimer at entry and at exit
#define TC_STAMP(i) do { if (threadIdx.x == 0) { unsigned long long g_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g_)); \
    g_tc_clock[blockIdx.x * 4 + 2 * (i)] = clock64(); g_tc_clock[blockIdx.x * 4 + 2 * (i) + 1] = (long long)g_; } } while (0)
#else
#define TC_STAMP(i)
#define TC_LAP_INIT
#define TC_LAP(var)
#define TC_REC(slot, var)
#endif

namespace {

using namespace tc;

constexpr int BLOCK_M = 128;
constexpr int EPI_WARPS = 16;
constexpr int NUM_THREADS = 64 + EPI_WARPS * 32; // 1 TMA warp + 1 MMA warp + 16 epilogue warps
constexpr int MAX_STAGES = 12;
constexpr int MAX_ACC = 4;

struct TcParams {
    int M, N, K;    // rows per matrix, output channels, reduction length
    int batch;      // independent matrices (1 unless every image has its own filter)
    int block_n, n_tiles, m_tiles;
    int swz;        // bytes of K per stage row: 32, 64 or 128
    int k_blocks;   // ceil(K / swz)
    int stages;
    int acc_stages; // TMEM accumulator buffers: 4 or 2 (int8), 1 (int16)
    int tmem_cols;  // power of two >= 32
    int out_pw;     // staged epilogue: bytes per row of a group's output piece (0 = rows are stored directly)
    int out_mask;   // swizzle mask of the staging tiles (7, 3, 1, 0)
    void *out;
    long long ops;  // output row stride in elements
    const int8_t *res; // optional residual added to the result (same rows as the output), or null
    long long rps;     // residual row stride in elements
    long long peer_delta[7]; // byte distance from `out` to the same buffer on other GPUs: every result row is stored there too
    int n_peer;
    unsigned *sched; // {next tile, CTAs done}: the tiles from static_tiles on are handed out by this counter; null = fixed walk
    int static_tiles; // tiles walked in the fixed order (a multiple of the grid size; all of them without a counter)
    EpiConfig epi;
};

constexpr int TILE_RING = 32; // tile numbers on their way from the producer to the MMA issuer (more than stages + accumulators)

// Epilogue of one int8 tile for outputs that cannot go through the staged path (piece widths that are not whole
// 16-byte groups, unaligned rows, channels outside the fast form): rows are stored directly from registers.  Out of
// line on purpose: the staged path in the kernel then carries none of this code's registers.
__device__ __noinline__ void epilogue_direct_tile(const TcParams &p, const FastParam *fast_s, uint32_t fp_base, uint32_t t0, long long m, int n0,
                                                  bool row_ok, bool fast, int parts, int part, bool allow_wide = true, uint32_t tbl = 0u)
{
    int8_t *orow = (int8_t *)p.out + m * p.ops + n0;
    const bool vec_ok = (p.ops % 16 == 0) && ((((uintptr_t)p.out) + n0) % 16 == 0);
    // what every row start (and every 16-column step from it) is aligned to
    const uintptr_t amix = (uintptr_t)p.ops | (((uintptr_t)p.out) + (uintptr_t)n0) | 16u;
    const int out_align = (int)(amix & (~amix + 1));
    if (fast && !tbl && vec_ok && p.N % 16 == 0 && !p.res && p.n_peer == 0) {
        // whole 16-column groups, aligned rows, one-add-one-shift constants
        const bool wide = allow_wide && (p.ops % 32 == 0) && ((((uintptr_t)p.out) + n0) % 32 == 0);
        const uint32_t fp = fp_base + (uint32_t)n0 * 8u;
        const int ncols = min(p.block_n, p.N - n0);
        if (p.epi.relu)
            epilogue_lean<true>(t0, fp, orow, ncols, parts, part, row_ok, wide);
        else
            epilogue_lean<false>(t0, fp, orow, ncols, parts, part, row_ok, wide);
        return;
    }
    int chunk = 0;
    for (int c0 = 0; c0 < p.block_n; c0 += 32, chunk++) {
        if (chunk % parts != part)
            continue;
        const bool two = c0 + 32 <= p.block_n;
        int32_t v[32];
        ld16(t0 + c0, v);
        if (two)
            ld16(t0 + c0 + 16, v + 16);
        ld_wait16(v);
        tie16(v + 16);
        uint32_t pk[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (fast) {
            if (p.epi.relu) {
                requant16_fast<true>(v, fast_s + n0 + c0, pk);
                if (two)
                    requant16_fast<true>(v + 16, fast_s + n0 + c0 + 16, pk + 4);
            } else {
                requant16_fast<false>(v, fast_s + n0 + c0, pk);
                if (two)
                    requant16_fast<false>(v + 16, fast_s + n0 + c0 + 16, pk + 4);
            }
            if (tbl) { // a fused table on rows that leave unstaged (`tbl`: its shared-memory copy): same lookups on the packed words
#pragma unroll
                for (int q = 0; q < 8; q++) pk[q] = lut4(pk[q], tbl);
            }
        } else {
            requant16_general(v, p.epi, n0 + c0, p.N, pk);
            if (two)
                requant16_general(v + 16, p.epi, n0 + c0 + 16, p.N, pk + 4);
        }
        if (row_ok) {
            const int count = min(two ? 32 : 16, p.N - (n0 + c0));
            if (count > 0 && p.res) { // folded Add: saturating byte sums with the residual's row
                const int8_t *rrow = p.res + m * p.rps + n0 + c0;
#pragma unroll
                for (int j = 0; j < 32; j++)
                    if (j < count) {
                        const int sum = (int)(int8_t)(pk[j >> 2] >> (8 * (j & 3))) + (int)rrow[j];
                        pk[j >> 2] = (pk[j >> 2] & ~(0xffu << (8 * (j & 3)))) | (((uint32_t)max(-128, min(127, sum)) & 0xffu) << (8 * (j & 3)));
                    }
            }
            // copies of the rows in other GPUs' memory (peer-mapped pointers): plain stores, the same words
            for (int pi = 0; pi < p.n_peer && count > 0; pi++) {
                int8_t *prow = orow + c0 + p.peer_delta[pi];
                store_bytes(prow, pk, min(count, 16), out_align);
                if (count > 16)
                    store_bytes(prow + 16, pk + 4, count - 16, out_align);
            }
            if (count > 0 && allow_wide) {
                store_bytes(orow + c0, pk, count, out_align);
            } else if (count > 0) {
                store_bytes(orow + c0, pk, min(count, 16), out_align);
                if (count > 16)
                    store_bytes(orow + c0 + 16, pk + 4, count - 16, out_align);
            }
        }
    }
}

template <bool I16>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_a_lo, const __grid_constant__ CUtensorMap map_b_lo,
               const __grid_constant__ CUtensorMap map_out, const __grid_constant__ TcParams p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int NPLANE = I16 ? 2 : 1;
    constexpr int NACC = I16 ? 3 : 1;
    const int a_bytes = BLOCK_M * p.swz;
    const int b_bytes = p.block_n * p.swz;
    const int stage_bytes = NPLANE * (a_bytes + b_bytes);
    const int n_pad = p.n_tiles * p.block_n;
    uint8_t *out_stage = smem + (size_t)p.stages * stage_bytes; // 4 tiles of [128][out_pw] bytes, 1024-byte aligned each
    const int out_tile_bytes = (BLOCK_M * p.out_pw + 1023) & ~1023;
    uint8_t *aux = out_stage + 4 * (size_t)out_tile_bytes;
    FastParam *fast_s = (FastParam *)aux; // n_pad entries, 16-byte aligned (block_n % 16 == 0)
    uint64_t *bars = (uint64_t *)(aux + sizeof(FastParam) * (size_t)n_pad);
    uint64_t *full_bar = bars, *empty_bar = bars + MAX_STAGES, *tfull_bar = bars + 2 * MAX_STAGES, *tempty_bar = tfull_bar + MAX_ACC;
    uint32_t *tmem_slot = (uint32_t *)(tempty_bar + MAX_ACC);
    int *slow_flag = (int *)(tmem_slot + 1);
    uint8_t *lut_s = (uint8_t *)(slow_flag + 3); // the fused 8-bit table, 256 bytes, 16-byte aligned
    volatile int *tile_ring = (volatile int *)(lut_s + 256); // TILE_RING tile numbers, producer -> MMA issuer
    volatile int *epi_tile = tile_ring + TILE_RING;          // MAX_ACC tile numbers, MMA issuer -> the accumulator's epilogue groups

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    TC_STAMP(0);
    const int total_tiles = p.batch * p.m_tiles * p.n_tiles;
    const int parts = 4 / p.acc_stages; // epilogue groups that share one tile (they split its columns)
    // Tiles are numbered n-fastest: tile = row_tile * n_tiles + n_tile with row_tile running over batch x m_tiles.  A CTA
    // starts with tile blockIdx.x; every further tile comes from a global counter (p.sched), so that an SM that runs
    // slower than the others (measured: one in ten takes 15-25 % longer per tile) gets fewer tiles instead of setting
    // the kernel's duration.  The producer fetches the numbers and passes them on through shared memory: to the MMA
    // issuer in a ring (published by the arrive on the first stage's "full" barrier), from there to the epilogue groups
    // (published by a plain arrive on the accumulator's "full" barrier, which therefore counts two arrivals: that one
    // and the tensor cores' commit).  A negative number ends the walk.

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < MAX_ACC; a++) {
            mbar_init(smem_u32(&tfull_bar[a]), 2);
            mbar_init(smem_u32(&tempty_bar[a]), 4 * parts);
        }
        *slow_flag = 0;
        fence_barrier_init();
    }
    if (threadIdx.x == 32 * 2) { // an epilogue thread: the descriptors are in the cache when the first copies are issued
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        if (I16) {
            prefetch_tensormap(&map_a_lo);
            prefetch_tensormap(&map_b_lo);
        } else if (p.out_pw) {
            prefetch_tensormap(&map_out);
        }
    }
    if (warp == 1)
        tmem_alloc(smem_u32(tmem_slot), p.tmem_cols);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // Per-channel constants for every output channel, once per kernel, by all threads: {bias_half, shift} pairs.
    bool fast = false;
    if (!I16) {
        stage_fast_params(p.epi, fast_s, p.N, n_pad, (int)threadIdx.x, NUM_THREADS, slow_flag);
        if (p.epi.lut)
            stage_lut(p.epi.lut, lut_s, (int)threadIdx.x, NUM_THREADS);
        __syncthreads();
        fast = !*slow_flag && !p.epi.half_even && !p.epi.lut_stride && p.K <= 32768; // one table rides on the staged form and on the packed words of unstaged rows; per-channel tables take the general path
    }
    // This CTA is set up (everything above reads launch parameters and model constants only): the next kernel's CTAs may
    // take SMs as they become free.  The producer below waits for the previous kernel before its first load, and every
    // other role only ever acts on what the producer brought in.
    if (threadIdx.x == 0)
        grid_dep_launch();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        // One lane runs the loop and issues the copies.  (Letting the whole warp walk the tiles and wait, with lane 0
        // issuing, measured the same on the network's short reductions and 25-35 % slower on the long reductions of a
        // large Gemm, where the issue rate of this loop and of the MMA loop below is what bounds the kernel.)
        const bool issuer = lane == 0;
        if (issuer) {
        grid_dep_wait(); // the previous kernel's output, and its use of the tile counter, before the first load
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        long long w_empty = 0, w_load = 0;
        (void)w_empty, (void)w_load;
        TC_LAP_INIT;
        // Tiles below p.static_tiles are walked in the fixed order (blockIdx.x, + gridDim.x, ...); the rest is handed out
        // by the counter, one number per tile and asked for one tile ahead (an atomic on a word that every SM hammers
        // takes ~1000 cycles to answer: with every tile handed out that way the producer no longer ran ahead)
        int tile = blockIdx.x; // the grid never has more CTAs than there are tiles
        bool handed = false;
        auto after = [&](int cur) {
            if (!handed && cur + (int)gridDim.x < p.static_tiles)
                return cur + (int)gridDim.x;
            if (!p.sched)
                return handed || cur + (int)gridDim.x >= total_tiles ? total_tiles : cur + (int)gridDim.x;
            handed = true;
            return p.static_tiles + (int)atomicAdd(p.sched, 1u);
        };
        int next = after(tile);
        int local = 0;
        for (; tile < total_tiles && ok; local++) {
            tile_ring[local & (TILE_RING - 1)] = tile;
            const int rows = tile / p.n_tiles, nt = tile - rows * p.n_tiles;
            const int bi = p.batch == 1 ? 0 : rows / p.m_tiles;
            const int m0 = (p.batch == 1 ? rows : rows % p.m_tiles) * BLOCK_M;
            const int n0 = nt * p.block_n;
            for (int kb = 0; kb < p.k_blocks; kb++) {
                TC_LAP(w_load);
                if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1)) {
                    ok = false;
                    break;
                }
                TC_LAP(w_empty);
                const uint32_t bar = smem_u32(&full_bar[stage]);
                const uint32_t st = smem_u32(smem) + (uint32_t)(stage * stage_bytes);
                mbar_arrive_expect_tx(bar, (uint32_t)stage_bytes);
                tma_load_3d(st, &map_a, kb * p.swz, m0, bi, bar);
                tma_load_3d(st + NPLANE * a_bytes, &map_b, kb * p.swz, n0, bi, bar);
                if (I16) {
                    tma_load_3d(st + a_bytes, &map_a_lo, kb * p.swz, m0, bi, bar);
                    tma_load_3d(st + 2 * a_bytes + b_bytes, &map_b_lo, kb * p.swz, n0, bi, bar);
                }
                if (++stage == p.stages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            // the number after next is asked for one tile ahead of its use: the answer is back long before it is needed
            tile = next;
            if (tile < total_tiles)
                next = after(tile);
        }
        if (ok) {
            // end of the walk: one stage without data whose ring entry is negative
            tile_ring[local & (TILE_RING - 1)] = -1;
            if (mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1))
                mbar_arrive(smem_u32(&full_bar[stage]));
            else
                ok = false;
        }
        if (!ok)
            atomicExch(&g_tc_error, ESPDL_ERR_TIMEOUT);
        TC_REC(0, w_empty);
        TC_REC(1, w_load);
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // One lane runs the loop and issues (see the producer).  Each tcgen05.mma of M = 128 costs this thread about 250
        // cycles whatever N is (measured with the role cycle counters: 4 MMAs per tile of K = 128 take ~1000 cycles), so
        // tiles are made as wide as TMEM allows and carry as few K steps as the layer has.
        const bool issuer = lane == 0;
        if (issuer) {
        int stage = 0;
        uint32_t phase = 0;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        long long w_tempty = 0, w_full = 0, w_issue = 0;
        (void)w_tempty, (void)w_full, (void)w_issue;
        TC_LAP_INIT;
        const uint32_t idesc_ss = idesc_i8(1, 1, BLOCK_M, p.block_n);
        const uint32_t idesc_su = idesc_i8(1, 0, BLOCK_M, p.block_n);
        const uint32_t idesc_us = idesc_i8(0, 1, BLOCK_M, p.block_n);
        const uint32_t idesc_uu = idesc_i8(0, 0, BLOCK_M, p.block_n);
        const int ksteps = p.swz / 32;
        const int last_ksteps = (p.K - (p.k_blocks - 1) * p.swz + 31) / 32; // 32-byte K steps of the last block that hold data
        const uint32_t smem_base = smem_u32(smem);
        for (int local = 0; ok; local++) {
            TC_LAP(w_issue);
            // the tile's first stage: its arrival publishes the tile number
            if (!mbar_wait(smem_u32(&full_bar[stage]), phase)) {
                ok = false;
                break;
            }
            TC_LAP(w_full);
            const int tile = tile_ring[local & (TILE_RING - 1)];
            if (tile < 0) {
                // end of the walk: every accumulator's epilogue groups are told, in the order they wait
                for (int a = 0; a < p.acc_stages && ok; a++) {
                    if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1)) {
                        ok = false;
                        break;
                    }
                    epi_tile[acc] = -1;
                    mbar_arrive(smem_u32(&tfull_bar[acc]));
                    mbar_arrive(smem_u32(&tfull_bar[acc]));
                    if (++acc == p.acc_stages) {
                        acc = 0;
                        acc_phase ^= 1;
                    }
                }
                break;
            }
            if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1)) {
                ok = false;
                break;
            }
            TC_LAP(w_tempty);
            fence_after();
            epi_tile[acc] = tile;
            const uint32_t d0 = tmem_base + (uint32_t)(acc * NACC * p.block_n);
            for (int kb = 0; kb < p.k_blocks; kb++) {
                TC_LAP(w_issue);
                if (kb != 0 && !mbar_wait(smem_u32(&full_bar[stage]), phase)) {
                    ok = false;
                    break;
                }
                TC_LAP(w_full);
                fence_after();
                const uint32_t st = smem_base + (uint32_t)(stage * stage_bytes);
                const uint64_t da = smem_desc_swizzled(st, p.swz);
                const uint64_t db = smem_desc_swizzled(st + NPLANE * a_bytes, p.swz);
                // the reduction's last block may end early: its K steps past the end would multiply the TMA unit's zero fill
                const int ks = kb == p.k_blocks - 1 ? last_ksteps : ksteps;
                if (!I16) {
                    const uint32_t first = kb != 0 ? 1u : 0u;
                    mma_i8(d0, da, db, idesc_ss, first);
                    if (ks > 1)
                        mma_i8(d0, da + 2, db + 2, idesc_ss, 1u);
                    if (ks > 2)
                        mma_i8(d0, da + 4, db + 4, idesc_ss, 1u);
                    if (ks > 3)
                        mma_i8(d0, da + 6, db + 6, idesc_ss, 1u);
                    commit(smem_u32(&empty_bar[stage]));
                } else {
                    const uint64_t da_lo = smem_desc_swizzled(st + a_bytes, p.swz);
                    const uint64_t db_lo = smem_desc_swizzled(st + 2 * a_bytes + b_bytes, p.swz);
                    for (int k = 0; k < ks; k++) {
                        const uint32_t accum = (kb | k) != 0;
                        const uint64_t koff = (uint64_t)(k * 2); // 32 bytes of K, in 16-byte units
                        mma_i8(d0, da + koff, db + koff, idesc_ss, accum);                      // hi * hi
                        mma_i8(d0 + p.block_n, da + koff, db_lo + koff, idesc_su, accum);       // hi * lo
                        mma_i8(d0 + p.block_n, da_lo + koff, db + koff, idesc_us, 1u);          // lo * hi
                        mma_i8(d0 + 2 * p.block_n, da_lo + koff, db_lo + koff, idesc_uu, accum); // lo * lo
                    }
                    commit(smem_u32(&empty_bar[stage]));
                }
                if (++stage == p.stages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (!ok)
                break;
            commit(smem_u32(&tfull_bar[acc]));
            mbar_arrive(smem_u32(&tfull_bar[acc])); // publishes epi_tile[acc]
            if (++acc == p.acc_stages) {
                acc = 0;
                acc_phase ^= 1;
            }
        }
        if (!ok)
            atomicExch(&g_tc_error, ESPDL_ERR_TIMEOUT);
        TC_REC(2, w_tempty);
        TC_REC(3, w_full);
        TC_REC(4, w_issue);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..17)
        const int ew = warp - 2;
        const int group = ew >> 2;               // 0..3
        const int acc = group % p.acc_stages;    // accumulator buffer this group reads
        const int part = group / p.acc_stages;   // which share of the tile's columns
        const int lane_group = warp & 3;         // TMEM lanes this warp may read: 32*lane_group .. +31
        const int row_in_tile = lane_group * 32 + lane;

        const uint32_t fp_base = epi_param_base(fast_s);
        uint32_t acc_phase = 0;
        bool ok = true;
        long long w_tfull = 0, w_work = 0, w_store = 0;
        (void)w_tfull, (void)w_work, (void)w_store;
        TC_LAP_INIT;
        while (ok) {
            TC_LAP(w_work);
            if (!mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase)) {
                ok = false;
                break;
            }
            TC_LAP(w_tfull);
            const int tile = epi_tile[acc];
            if (tile < 0)
                break;
            const int rows = tile / p.n_tiles, nt = tile - rows * p.n_tiles;
            const int bi = p.batch == 1 ? 0 : rows / p.m_tiles;
            const int m0 = (p.batch == 1 ? rows : rows % p.m_tiles) * BLOCK_M;
            const int n0 = nt * p.block_n;
            acc_phase ^= 1;
            fence_after();
            const bool row_ok = m0 + row_in_tile < p.M;
            const long long m = (long long)bi * p.M + m0 + row_in_tile; // row of the output tensor
            const uint32_t t0 = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(acc * NACC * p.block_n);
            if (!I16) {
                if (fast && p.out_pw) {
                    // staged: requantise into this group's shared-memory tile, one TMA store per piece
                    const bool leader = (ew & 3) == 0 && lane == 0;
                    const uint32_t buf = smem_u32(out_stage + (size_t)group * out_tile_bytes);
                    if (leader)
                        bulk_wait_read_all(); // the previous store out of this tile has been read
                    named_bar(2 + group, 128);
                    TC_LAP(w_store);
                    const int col0 = part * p.out_pw;
                    const uint32_t fpp = fp_base + (uint32_t)(n0 + col0) * 8u;
                    const int floor_q = p.epi.relu ? 0 : INT_MIN;
                    if (p.epi.lut) {
                        epilogue_stage_lut(t0 + col0, fpp, buf, row_in_tile, p.out_pw, (uint32_t)p.out_mask, floor_q, smem_u32(lut_s));
                    } else if (p.res)
                        epilogue_stage_residual(t0 + col0, fpp, buf, row_in_tile, p.out_pw, (uint32_t)p.out_mask, floor_q,
                                                p.res + m * p.rps + n0 + col0, row_ok, p.N - (n0 + col0));
                    else if (p.out_pw == 128)
                        epilogue_stage<128>(t0 + col0, fpp, buf, row_in_tile, 128, floor_q);
                    else if (p.out_pw == 96)
                        epilogue_stage<96>(t0 + col0, fpp, buf, row_in_tile, 96, floor_q);
                    else if (p.out_pw == 64)
                        epilogue_stage<64>(t0 + col0, fpp, buf, row_in_tile, 64, floor_q);
                    else
                        epilogue_stage<0>(t0 + col0, fpp, buf, row_in_tile, p.out_pw, floor_q);
                    // the accumulator is free as soon as this warp's TMEM loads are done: hand it back before the
                    // shared-memory tile is completed and stored, so that the MMAs of the tile after next start earlier
                    fence_before();
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(smem_u32(&tempty_bar[acc]));
                    fence_async_smem();
                    named_bar(2 + group, 128);
                    if (leader) {
                        tma_store_3d(&map_out, buf, n0 + col0, m0, bi); // rows >= M and columns >= N are clipped
                        bulk_commit();
                    }
                    continue;
                }
                epilogue_direct_tile(p, fast_s, fp_base, t0, m, n0, row_ok, fast, parts, part, true, p.epi.lut ? smem_u32(lut_s) : 0u);
            } else {
                int chunk = 0;
                for (int c0 = 0; c0 < p.block_n; c0 += 16, chunk++) {
                    if (chunk % parts != part)
                        continue;
                    int32_t vh[16], vm[16], vl[16];
                    ld16(t0 + c0, vh);
                    ld16(t0 + p.block_n + c0, vm);
                    ld16(t0 + 2 * p.block_n + c0, vl);
                    ld_wait16(vh);
                    tie16(vm);
                    tie16(vl);
                    if (row_ok && n0 + c0 < p.N) {
                        int16_t *op = (int16_t *)p.out + m * p.ops + n0 + c0;
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const int n = n0 + c0 + j;
                            if (n < p.N) {
                                const long long a = ((long long)vh[j] << 16) + ((long long)vm[j] << 8) + (long long)vl[j];
                                const int e = p.epi.per_channel ? __ldg(p.epi.ew + n) : p.epi.ew_scalar;
                                const int shift = max(-62, min(62, p.epi.e_shift_base - e));
                                const long long b = p.epi.bias ? __ldg((const long long *)p.epi.bias + n) : 0ll;
                                op[j] = (int16_t)requant16(a, b, shift, p.epi.relu, p.epi.half_even);
                            }
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
            atomicExch(&g_tc_error, ESPDL_ERR_TIMEOUT);
        if (ew == 0 && lane == 0) {
            TC_LAP(w_work);
            TC_REC(5, w_tfull);
            TC_REC(6, w_work);
            TC_REC(7, w_store);
        }
        if (!I16 && p.out_pw && (ew & 3) == 0 && lane == 0)
            bulk_wait_all(); // shared memory stays allocated until the last store has left it
    }

    fence_before();
    __syncthreads();
    TC_STAMP(1);
    if (warp == 1) {
        fence_after();
        tmem_dealloc(tmem_base, p.tmem_cols);
    }
    // the last CTA to get here leaves the counters as it found them (thread 0 is also the one that asked for tiles)
    if (p.sched && threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(p.sched + 1, 1u) == gridDim.x - 1) {
            p.sched[0] = 0;
            p.sched[1] = 0;
        }
    }
}

// ------------------------------------------------------------------------------------------ CTA pairs (large int8 Gemm)
// For a reduction long enough to be bound by the tensor pipe, the tile above needs (128 + 256) * 128 bytes per 4 MMA
// steps and SM; the bytes a shared memory can keep in flight then cover less than the load latency and the tensor
// pipe idles about half of the time (measured: 45 % active at 65536x1024x1024).  Here two CTAs of a cluster (the two
// SMs of a TPC) work on one 256 x block_n tile with tcgen05.mma.cta_group::2: each loads its own 128 rows of A and only
// HALF of the B tile (the tensor cores read the other half from the peer's shared memory), i.e. a third fewer bytes
// per MMA and SM, so the same shared memory holds half as many more stages.  The even CTA of the pair issues the MMAs
// for both; barriers: every TMA load of either CTA completes bytes on the even CTA's "full" barrier, the MMA
// issuer's commits arrive on both CTAs' "empty" and "accumulator full" barriers (one commit per CTA, addressed with
// mapa), both CTAs' epilogue warps arrive on the even CTA's "accumulator empty" barrier.  Epilogue: direct row stores.
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory variable in the CTA with rank `rank`
__device__ __forceinline__ uint32_t mapa_rank(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t leader_bar)
{
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
                 "l"(map), "r"(leader_bar), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void mma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    const uint32_t z = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(z)
        : "memory");
}
__device__ __forceinline__ void commit_pair(uint32_t cluster_bar)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t base, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b_half, const TcParams p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int a_bytes = BLOCK_M * p.swz;
    const int bh_bytes = (p.block_n / 2) * p.swz;
    const int stage_bytes = a_bytes + bh_bytes;
    const int n_pad = p.n_tiles * p.block_n;
    uint8_t *aux = smem + (size_t)p.stages * stage_bytes;
    FastParam *fast_s = (FastParam *)aux;
    uint64_t *bars = (uint64_t *)(aux + sizeof(FastParam) * (size_t)n_pad);
    uint64_t *full_bar = bars, *empty_bar = bars + MAX_STAGES, *tfull_bar = bars + 2 * MAX_STAGES, *tempty_bar = tfull_bar + MAX_ACC;
    uint32_t *tmem_slot = (uint32_t *)(tempty_bar + MAX_ACC);
    int *slow_flag = (int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair_m_tiles = (p.m_tiles + 1) / 2;
    const int total_pairs = pair_m_tiles * p.n_tiles;
    const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int parts = 4 / p.acc_stages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < MAX_ACC; a++) {
            mbar_init(smem_u32(&tfull_bar[a]), 1);
            mbar_init(smem_u32(&tempty_bar[a]), 2 * 4 * parts); // the epilogue warps of both CTAs
        }
        *slow_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1)
        tmem_alloc_pair(smem_u32(tmem_slot), p.tmem_cols); // the same warp of both CTAs, the same slot address
    fence_before();
    __syncthreads();
    cluster_sync_all(); // both CTAs' barriers exist before either touches the other's
    fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = pair_id; t < total_pairs && ok; t += n_pairs) {
                const int m0 = (t / p.n_tiles) * 2 * BLOCK_M + (int)rank * BLOCK_M;
                const int n0 = (t % p.n_tiles) * p.block_n + (int)rank * (p.block_n / 2);
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1)) {
                        ok = false;
                        break;
                    }
                    if (rank == 0)
                        mbar_arrive_expect_tx(smem_u32(&full_bar[stage]), (uint32_t)(2 * stage_bytes)); // the bytes of both CTAs
                    const uint32_t bar = mapa_rank(smem_u32(&full_bar[stage]), 0);
                    uint8_t *st = smem + (size_t)stage * stage_bytes;
                    tma_load_3d_pair(smem_u32(st), &map_a, kb * p.swz, m0, 0, bar);
                    tma_load_3d_pair(smem_u32(st + a_bytes), &map_b_half, kb * p.swz, n0, 0, bar);
                    if (++stage == p.stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok)
                atomicExch(&g_tc_error, ESPDL_ERR_TIMEOUT);
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (even CTA only)
        if (lane == 0 && rank == 0) {
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            const uint32_t idesc = idesc_i8(1, 1, 2 * BLOCK_M, p.block_n);
            const int ksteps = p.swz / 32;
            for (int t = pair_id; t < total_pairs && ok; t += n_pairs) {
                if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1)) {
                    ok = false;
                    break;
                }
                fence_after();
                const uint32_t d0 = tmem_base + (uint32_t)(acc * p.block_n);
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    if (!mbar_wait(smem_u32(&full_bar[stage]), phase)) {
                        ok = false;
                        break;
                    }
                    fence_after();
                    const uint32_t st = smem_u32(smem + (size_t)stage * stage_bytes);
                    const uint64_t da = smem_desc_swizzled(st, p.swz);
                    const uint64_t db = smem_desc_swizzled(st + a_bytes, p.swz);
                    for (int k = 0; k < ksteps; k++) mma_i8_pair(d0, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0);
                    commit_pair(mapa_rank(smem_u32(&empty_bar[stage]), 0));
                    commit_pair(mapa_rank(smem_u32(&empty_bar[stage]), 1));
                    if (++stage == p.stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok)
                    break;
                commit_pair(mapa_rank(smem_u32(&tfull_bar[acc]), 0));
                commit_pair(mapa_rank(smem_u32(&tfull_bar[acc]), 1));
                if (++acc == p.acc_stages) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
            if (!ok)
                atomicExch(&g_tc_error, ESPDL_ERR_TIMEOUT);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..17 of both CTAs)
        const int ew = warp - 2;
        const int group = ew >> 2;
        const int acc = group % p.acc_stages;
        const int part = group / p.acc_stages;
        const int lane_group = warp & 3;
        const int row_in_tile = lane_group * 32 + lane;
        const int et = threadIdx.x - 64;
        stage_fast_params(p.epi, fast_s, p.N, n_pad, et, EPI_WARPS * 32, slow_flag);
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
        const bool fast = !*slow_flag && !p.epi.half_even && !p.epi.lut && p.K <= 32768;
        const uint32_t fp_base = epi_param_base(fast_s);
        const uint32_t tempty_leader = mapa_rank(smem_u32(&tempty_bar[acc]), 0);
        uint32_t acc_phase = 0;
        bool ok = true;
        int local = 0;
        for (int t = pair_id; t < total_pairs && ok; t += n_pairs, local++) {
            if (local % p.acc_stages != acc)
                continue;
            const int m0 = (t / p.n_tiles) * 2 * BLOCK_M + (int)rank * BLOCK_M;
            const int n0 = (t % p.n_tiles) * p.block_n;
            if (!mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase)) {
                ok = false;
                break;
            }
            acc_phase ^= 1;
            fence_after();
            const bool row_ok = m0 + row_in_tile < p.M;
            const long long m = (long long)m0 + row_in_tile;
            const uint32_t t0 = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(acc * p.block_n);
            // 128-bit stores: in this kernel the 256-bit form stored only the first word of each 32 bytes
            epilogue_direct_tile(p, fast_s, fp_base, t0, m, n0, row_ok, fast, parts, part, false);
            fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive_cluster(tempty_leader);
        }
        if (!ok && lane == 0)
            atomicExch(&g_tc_error, ESPDL_ERR_TIMEOUT);
    }

    fence_before();
    __syncthreads();
    cluster_sync_all(); // neither CTA leaves (or frees TMEM) while the other may still read its shared memory or barriers
    if (warp == 1) {
        fence_after();
        tmem_dealloc_pair(tmem_base, p.tmem_cols);
    }
}

// int16 [rows][K] (row stride `stride` elements) -> dense byte planes hi (signed) and lo (unsigned).
__global__ void __launch_bounds__(256) split_limbs_kernel(const int16_t *__restrict__ src, long long stride, int K, long long total,
                                                          int8_t *__restrict__ hi, uint8_t *__restrict__ lo)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / K;
        const int k = (int)(i % K);
        const int v = src[r * stride + k];
        hi[i] = (int8_t)(v >> 8);
        lo[i] = (uint8_t)(v & 0xff);
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// uint8 tensor [mats][rows][cols] with `row_stride` bytes between rows and `mat_stride` bytes between matrices;
// box = 1 x box_rows x box_cols.
int make_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint64_t row_stride, uint32_t box_rows,
             uint32_t box_cols, int swz, uint64_t mats = 1, uint64_t mat_stride = 0)
{
    EncodeTiledFn enc = get_encode();
    if (!enc)
        return set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point not found");
    if (mats <= 1)
        mat_stride = (rows * row_stride + 15) / 16 * 16; // unused with a single matrix, but it must be a legal stride
    cuuint64_t dims[3] = {cols, rows, mats ? mats : 1};
    cuuint64_t strides[2] = {row_stride, mat_stride};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapSwizzle sw = swz == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
        : (swz == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : (swz == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE));
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
        return ESPDL_ERR_CUDA;
    }
    return ESPDL_OK;
}

// Bytes of K per stage row (= TMA box width = swizzle width).  Wide rows move fastest through the TMA unit, so
// 128 is used as soon as K fills three quarters of such a row; columns past K are zero-filled, not fetched.
int pick_swz(int K)
{
    if (K >= 96)
        return 128;
    if (K > 32)
        return 64;
    return 32;
}

constexpr size_t SMEM_BUDGET = 200 * 1024;      // stages + staging tiles of the layers whose epilogue is staged
constexpr size_t SMEM_BUDGET_DEEP = 225 * 1024; // long reductions with direct row stores: one more stage in flight (1.79 -> 1.97 POPS
                                                // at 65536x1024x1024); for the staged layers the larger budget measured 5 % slower

size_t aux_bytes(const TcParams &p)
{
    return sizeof(FastParam) * (size_t)p.n_tiles * p.block_n + (2 * MAX_STAGES + 2 * MAX_ACC) * 8 + 32 + 256 + (TILE_RING + MAX_ACC) * 4;
}

bool plan(const espdl_conv_desc &d, TcParams &p, bool force_direct = false)
{
    const bool i16 = d.dtype == ESPDL_DTYPE_INT16;
    // one matrix over all pixels of all images, or - when every image has its own filter - one matrix per image
    const bool batched = d.filter_image_stride != 0;
    if (batched && (i16 || d.filter_image_stride % 16 != 0))
        return false;
    const long long M = (batched ? 1ll : (long long)d.n) * d.out_h * d.out_w;
    if (M > 0x7fffffffll || d.out_c > 8192)
        return false;
    p.M = (int)M, p.N = d.out_c, p.K = d.in_c;
    p.batch = batched ? d.n : 1;
    int max_bn = i16 ? 128 : 256;
    if (const char *cap = getenv("ESPDL_B200_MAX_BLOCK_N")) // tile width cap (a multiple of 16), for experiments
        max_bn = max(16, min(max_bn, atoi(cap) / 16 * 16));
    p.n_tiles = (p.N + max_bn - 1) / max_bn;
    p.block_n = (((p.N + p.n_tiles - 1) / p.n_tiles) + 15) / 16 * 16;
    if (!i16 && p.block_n > 128)
        p.block_n = (p.block_n + 31) / 32 * 32; // two epilogue groups split a wide tile into whole 16-byte pieces
    p.n_tiles = (p.N + p.block_n - 1) / p.block_n;
    p.m_tiles = (p.M + BLOCK_M - 1) / BLOCK_M;
    p.swz = pick_swz(p.K);
    p.k_blocks = (p.K + p.swz - 1) / p.swz;
    p.acc_stages = i16 ? 1 : (4 * p.block_n <= 512 ? 4 : 2);
    int cols = p.acc_stages * (i16 ? 3 : 1) * p.block_n;
    int pow2 = 32;
    while (pow2 < cols) pow2 *= 2;
    if (pow2 > 512)
        return false;
    p.tmem_cols = pow2;
    // staged epilogue (int8): each group of four epilogue warps owns a piece of block_n / parts columns
    const long long ops = d.out_pixel_stride ? d.out_pixel_stride : d.out_c;
    p.out_pw = 0, p.out_mask = 0;
    const long long rps = d.residual_pixel_stride ? d.residual_pixel_stride : d.out_c;
    const bool res_ok = !d.residual || (rps % 16 == 0 && ((uintptr_t)d.residual % 16) == 0);
    if (!i16 && ops % 16 == 0 && ((uintptr_t)d.output % 16) == 0 && res_ok && !force_direct && !getenv("ESPDL_B200_DIRECT_STORES")) {
        const int parts = 4 / p.acc_stages;
        if (p.block_n % (16 * parts) == 0 && p.block_n / parts <= 128) {
            p.out_pw = p.block_n / parts;
            p.out_mask = p.out_pw == 128 ? 7 : (p.out_pw == 64 ? 3 : 0);
        }
    }
    size_t out_bytes = 4 * (size_t)((BLOCK_M * p.out_pw + 1023) & ~1023);
    size_t stage_bytes = (size_t)(i16 ? 2 : 1) * (BLOCK_M + p.block_n) * p.swz;
    int stages = (int)((SMEM_BUDGET - aux_bytes(p) - out_bytes - 1024) / stage_bytes);
    // A wide tile with a reduction of two 128-byte blocks and room for only two or three stages has barely one tile's loads
    // in flight, and every tile then waits a full load latency (192 -> 256 columns over 3.3 M rows: 0.39 ms).  Blocks of 64
    // bytes make stages half as large: more of them, more tiles in flight (0.28 ms), although the TMA unit moves 64-byte
    // rows more slowly - so only where the 128-byte form is starved.
    if (!i16 && p.swz == 128 && p.k_blocks == 2 && stages < 3 * p.k_blocks / 2 + 1 && !getenv("ESPDL_B200_NO_NARROW_K")) {
        const size_t stage64 = (size_t)(BLOCK_M + p.block_n) * 64;
        const int kb64 = (p.K + 63) / 64;
        const int stages64 = (int)std::min<size_t>((SMEM_BUDGET - aux_bytes(p) - out_bytes - 1024) / stage64, MAX_STAGES);
        if (stages64 * p.k_blocks > stages * kb64) { // more tiles in flight
            p.swz = 64, p.k_blocks = kb64, stage_bytes = stage64, stages = stages64;
        }
    }
    if (p.out_pw && p.k_blocks > 2 && stages < 4) {
        // a long reduction needs the deep load pipeline more than the output needs staging
        p.out_pw = 0, p.out_mask = 0, out_bytes = 0;
        stages = (int)((SMEM_BUDGET_DEEP - aux_bytes(p) - 1024) / stage_bytes);
    }
    if (stages < 2)
        return false;
    p.stages = stages > MAX_STAGES ? MAX_STAGES : stages;
    return true;
}

// The CTA-pair kernel takes large int8 products without a per-image filter: long reductions, wide outputs, enough tiles.
bool pair_plan(const espdl_conv_desc &d, TcParams &p)
{
    // Off unless ESPDL_B200_CTA_PAIRS=1: measured slower than the one-CTA kernel so far (65536x1024x1024: 79 us against 70 us).
    const char *on = getenv("ESPDL_B200_CTA_PAIRS");
    if (d.dtype != ESPDL_DTYPE_INT8 || d.filter_image_stride != 0 || !on || atoi(on) == 0)
        return false;
    const long long M = (long long)d.n * d.out_h * d.out_w;
    if (M > 0x7fffffffll || d.out_c > 8192 || d.out_c < 256 || d.in_c < 512 || M < 2048)
        return false;
    p.M = (int)M, p.N = d.out_c, p.K = d.in_c, p.batch = 1;
    p.n_tiles = (p.N + 255) / 256;
    p.block_n = ((p.N + p.n_tiles - 1) / p.n_tiles + 31) / 32 * 32;
    p.n_tiles = (p.N + p.block_n - 1) / p.block_n;
    p.m_tiles = (p.M + BLOCK_M - 1) / BLOCK_M;
    p.swz = 128;
    p.k_blocks = (p.K + p.swz - 1) / p.swz;
    p.acc_stages = 2 * p.block_n <= 512 ? 2 : 1;
    if (p.acc_stages < 2)
        return false;
    p.tmem_cols = 512;
    p.out_pw = 0, p.out_mask = 0;
    const size_t stage_bytes = (size_t)(BLOCK_M + p.block_n / 2) * p.swz;
    const int stages = (int)((SMEM_BUDGET_DEEP - aux_bytes(p) - 1024) / stage_bytes);
    if (stages < 3)
        return false;
    p.stages = stages > MAX_STAGES ? MAX_STAGES : stages;
    return true;
}

int launch_pair(const espdl_conv_desc &d, TcParams &p, cudaStream_t s)
{
    const int ips = d.in_pixel_stride ? d.in_pixel_stride : d.in_c;
    CUtensorMap ma, mb;
    int st;
    if ((st = make_map(&ma, d.input, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)ips, BLOCK_M, (uint32_t)p.swz, p.swz, 1, (uint64_t)p.M * ips)))
        return st;
    if ((st = make_map(&mb, d.filter, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)p.K, (uint32_t)(p.block_n / 2), (uint32_t)p.swz, p.swz, 1, 0)))
        return st;
    const size_t stage_bytes = (size_t)(BLOCK_M + p.block_n / 2) * p.swz;
    const size_t smem = 1024 + (size_t)p.stages * stage_bytes + aux_bytes(p);
    static std::once_flag attr_once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(attr_once, [] { attr_err = cudaFuncSetAttribute(gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(SMEM_BUDGET_DEEP + 2048)); });
    if (attr_err != cudaSuccess)
        return set_cuda_error(attr_err, "cudaFuncSetAttribute(gemm_tc_pair_kernel)");
    const long long pairs = (long long)((p.m_tiles + 1) / 2) * p.n_tiles;
    const int grid = 2 * (int)min(pairs, (long long)(num_sms() / 2));
    gemm_tc_pair_kernel<<<grid, NUM_THREADS, smem, s>>>(ma, mb, p); // cluster size 2 is a compile-time attribute of the kernel
    count_launch();
    return check_launch("gemm_tc_pair");
}

} // namespace

bool conv2d_tc_supported(const espdl_conv_desc &d)
{
    if (d.group != 1 || d.kh != 1 || d.kw != 1 || d.stride_h != 1 || d.stride_w != 1)
        return false;
    if (d.pad_top || d.pad_bottom || d.pad_left || d.pad_right)
        return false;
    const int ips = d.in_pixel_stride ? d.in_pixel_stride : d.in_c;
    if (d.dtype == ESPDL_DTYPE_INT8) {
        if (d.in_c % 16 || ips % 16 || ((uintptr_t)d.input % 16) || ((uintptr_t)d.filter % 16))
            return false;
    } else {
        if (d.in_c % 16 || d.in_c > 16384) // planes are dense [rows][K] bytes: K % 16 keeps TMA strides legal
            return false;
    }
    TcParams p;
    return plan(d, p);
}

size_t conv2d_tc_workspace_bytes(const espdl_conv_desc &d)
{
    if (d.dtype != ESPDL_DTYPE_INT16)
        return 0;
    const size_t M = (size_t)d.n * d.out_h * d.out_w;
    const size_t a = (M * d.in_c + 255) / 256 * 256, b = ((size_t)d.out_c * d.in_c + 255) / 256 * 256;
    return 2 * a + 2 * b;
}

int conv2d_tc(const espdl_conv_desc &d, void *workspace, size_t workspace_bytes, cudaStream_t s, const long long *peer_delta, int n_peer)
{
    TcParams p;
    if (n_peer < 0 || n_peer > 7 || (n_peer > 0 && (d.dtype != ESPDL_DTYPE_INT8 || !peer_delta)))
        return ESPDL_ERR_UNSUPPORTED;
    if (!plan(d, p, n_peer > 0))
        return ESPDL_ERR_UNSUPPORTED;
    p.n_peer = n_peer;
    p.sched = nullptr, p.static_tiles = 0;
    for (int i = 0; i < 7; i++) p.peer_delta[i] = i < n_peer ? peer_delta[i] : 0;
    const bool i16 = d.dtype == ESPDL_DTYPE_INT16;
    const int ips = d.in_pixel_stride ? d.in_pixel_stride : d.in_c;
    p.out = d.output;
    p.ops = d.out_pixel_stride ? d.out_pixel_stride : d.out_c;
    p.res = (const int8_t *)d.residual;
    p.rps = d.residual_pixel_stride ? d.residual_pixel_stride : d.out_c;
    p.epi.bias = d.bias, p.epi.ew = d.filter_exponents, p.epi.lut = d.lut, p.epi.lut_stride = d.lut_channel_stride;
    p.epi.e_shift_base = d.out_exponent - d.in_exponent;
    p.epi.ew_scalar = d.filter_exponent, p.epi.per_channel = d.per_channel;
    p.epi.relu = d.activation == ESPDL_ACT_RELU, p.epi.half_even = d.round_mode == ESPDL_ROUND_HALF_EVEN;
    {
        TcParams pp = p;
        if (!i16 && n_peer == 0 && ips % 16 == 0 && pair_plan(d, pp))
            return launch_pair(d, pp, s);
    }

    CUtensorMap ma, mb, ma_lo, mb_lo;
    int st;
    if (!i16) {
        if ((st = make_map(&ma, d.input, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)ips, BLOCK_M, (uint32_t)p.swz, p.swz, (uint64_t)p.batch,
                           (uint64_t)p.M * ips)))
            return st;
        if ((st = make_map(&mb, d.filter, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)p.K, (uint32_t)p.block_n, (uint32_t)p.swz, p.swz, (uint64_t)p.batch,
                           (uint64_t)d.filter_image_stride)))
            return st;
        ma_lo = ma, mb_lo = mb;
    } else {
        const size_t a = ((size_t)p.M * p.K + 255) / 256 * 256, b = ((size_t)p.N * p.K + 255) / 256 * 256;
        if (workspace_bytes < 2 * a + 2 * b || !workspace || ((uintptr_t)workspace % 16))
            return ESPDL_ERR_INVALID_ARG;
        int8_t *a_hi = (int8_t *)workspace;
        uint8_t *a_lo = (uint8_t *)workspace + a;
        int8_t *b_hi = (int8_t *)workspace + 2 * a;
        uint8_t *b_lo = (uint8_t *)workspace + 2 * a + b;
        const long long ta = (long long)p.M * p.K, tb = (long long)p.N * p.K;
        const long long cap = (long long)num_sms() * 32;
        split_limbs_kernel<<<(unsigned)min((ta + 255) / 256, cap), 256, 0, s>>>((const int16_t *)d.input, ips, p.K, ta, a_hi, a_lo);
        split_limbs_kernel<<<(unsigned)min((tb + 255) / 256, cap), 256, 0, s>>>((const int16_t *)d.filter, p.K, p.K, tb, b_hi, b_lo);
        count_launch(2);
        if ((st = check_launch("split_limbs")))
            return st;
        if ((st = make_map(&ma, a_hi, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)p.K, BLOCK_M, (uint32_t)p.swz, p.swz)) ||
            (st = make_map(&ma_lo, a_lo, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)p.K, BLOCK_M, (uint32_t)p.swz, p.swz)) ||
            (st = make_map(&mb, b_hi, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)p.K, (uint32_t)p.block_n, (uint32_t)p.swz, p.swz)) ||
            (st = make_map(&mb_lo, b_lo, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)p.K, (uint32_t)p.block_n, (uint32_t)p.swz, p.swz)))
            return st;
    }
    const size_t stage_bytes = (size_t)(i16 ? 2 : 1) * (BLOCK_M + p.block_n) * p.swz;
    size_t smem = 1024 + (size_t)p.stages * stage_bytes + 4 * (size_t)((BLOCK_M * p.out_pw + 1023) & ~1023) + aux_bytes(p);
    CUtensorMap mo = ma;
    if (p.out_pw) {
        const int osw = p.out_pw == 128 ? 128 : (p.out_pw == 64 ? 64 : 0);
        if ((st = make_map(&mo, d.output, (uint64_t)p.M, (uint64_t)p.N, (uint64_t)p.ops, BLOCK_M, (uint32_t)p.out_pw, osw, (uint64_t)p.batch,
                           (uint64_t)p.M * (uint64_t)p.ops)))
            return st;
    }
    if (smem < 120 * 1024) // more than half an SM's shared memory: one CTA per SM, so TMEM allocation never waits on a neighbour
        smem = 120 * 1024;
    const long long all_tiles = (long long)p.batch * p.m_tiles * p.n_tiles;
    if (all_tiles > 0x7fffffffll)
        return ESPDL_ERR_TOO_LARGE;
    const int grid = (int)min(all_tiles, (long long)num_sms());
    // three quarters of the tiles in the fixed order, the last quarter to whichever SM is free
    p.sched = all_tiles >= 4ll * grid && all_tiles < (1ll << 30) ? sched_counters(s) : nullptr;
    p.static_tiles = p.sched ? (int)(all_tiles * 3 / 4 / grid) * grid : (int)all_tiles;
    static std::once_flag attr_once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(attr_once, [] {
        attr_err = cudaFuncSetAttribute(gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(SMEM_BUDGET_DEEP + 2048));
        if (attr_err == cudaSuccess)
            attr_err = cudaFuncSetAttribute(gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(SMEM_BUDGET_DEEP + 2048));
    });
    if (attr_err != cudaSuccess)
        return set_cuda_error(attr_err, "cudaFuncSetAttribute(gemm_tc_kernel)");
    if (i16)
        gemm_tc_kernel<true><<<grid, NUM_THREADS, smem, s>>>(ma, mb, ma_lo, mb_lo, mo, p);
    else
        launch_overlapped(gemm_tc_kernel<false>, dim3(grid), dim3(NUM_THREADS), smem, s, ma, mb, ma_lo, mb_lo, mo, p);
    count_launch();
    return check_launch("gemm_tc");
}

} // namespace espdl

// ------------------------------------------------------------------ allocation-free int16 Gemm / pointwise conv
// Fixed scratch for espdl_b200_gemm_s16_static: the byte planes of both int16 operands live in this array
// instead of a caller-provided or cached cudaMalloc buffer.  It is part of the library image, so every GPU
// that loads the library carries it until the process exits.
namespace espdl {
static __device__ __align__(256) unsigned char g_static_limb_scratch[ESPDL_B200_STATIC_SCRATCH_BYTES];
}

extern "C" int espdl_b200_gemm_s16_static(const espdl_conv_desc *desc, void *stream)
{
    using namespace espdl;
    // the same descriptor checks as espdl_b200_conv2d, before anything is planned or launched
    const int st = conv_validate(desc);
    if (st)
        return st;
    if (desc->dtype != ESPDL_DTYPE_INT16 || desc->lut || desc->residual || desc->filter_image_stride != 0 || !conv2d_tc_supported(*desc))
        return ESPDL_ERR_UNSUPPORTED;
    if (desc->n == 0)
        return ESPDL_OK;
    const size_t need = conv2d_tc_workspace_bytes(*desc);
    if (need > (size_t)ESPDL_B200_STATIC_SCRATCH_BYTES)
        return set_error_text(ESPDL_ERR_TOO_LARGE,
                              "espdl_b200_gemm_s16_static: %zu bytes of scratch needed, the fixed array holds %u; use "
                              "espdl_b200_conv2d_ws with a caller-owned buffer",
                              need, (unsigned)ESPDL_B200_STATIC_SCRATCH_BYTES);
    // In host code the array's name is only a handle; the device address comes from cudaGetSymbolAddress, asked
    // once per device with that device current.
    static void *addr_of_device[64] = {nullptr};
    static std::mutex addr_mutex;
    int dev = -1;
    ESPDL_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64)
        return ESPDL_ERR_NO_DEVICE;
    void *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(addr_mutex);
        if (!addr_of_device[dev]) {
            void *p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, g_static_limb_scratch);
            if (e != cudaSuccess)
                return set_cuda_error(e, "cudaGetSymbolAddress(g_static_limb_scratch)");
            addr_of_device[dev] = p;
        }
        scratch = addr_of_device[dev];
    }
    return conv2d_tc(*desc, scratch, (size_t)ESPDL_B200_STATIC_SCRATCH_BYTES, (cudaStream_t)stream);
}

#ifdef ESPDL_TC_TIMING
// Measurement builds only: copies the role cycle counters of the last gemm_tc_kernel launch (8 values per CTA).
extern "C" int espdl_b200_debug_gemm_timing(long long *out, int ctas)
{
    return cudaMemcpyFromSymbol(out, espdl::g_tc_timing, sizeof(long long) * 8 * (size_t)(ctas > 256 ? 256 : ctas)) == cudaSuccess ? 0 : -3;
}
extern "C" int espdl_b200_debug_gemm_clock(long long *out, int ctas)
{
    return cudaMemcpyFromSymbol(out, espdl::g_tc_clock, sizeof(long long) * 4 * (size_t)(ctas > 256 ? 256 : ctas)) == cudaSuccess ? 0 : -3;
}
#endif
