// Tensor-core (tcgen05) tile kernel for pointwise Conv2D / Gemm / MatMul, int8 and int16.
//
//   out[m, n] = epilogue( sum_k A[m, k] * W[n][k] + bias[n] )         m = pixel, n = output channel
//
// Replaces dl::base::conv2d<> for 1x1 filters (esp-dl/dl/base/dl_base_conv2d.cpp:9-60 conv2d_11cn,
// epilogue esp-dl/dl/base/dl_base_activate_buffer.hpp:27-73), which is also what Gemm and MatMul
// run (esp-dl/dl/module/include/dl_module_gemm.hpp:85-123).
//
// Structure (one persistent CTA per SM, 6 warps):
//   warp 0   TMA producer: cp.async.bulk.tensor 2-D tiles of A (128 rows x SWZ bytes of K) and of
//            W (BLOCK_N rows x SWZ bytes) into a ring of shared-memory stages, swizzled so that
//            the MMA reads them without bank conflicts; rows/columns past the tensor are zero-filled
//            by the TMA unit, so ragged M, N and K need no separate code.
//   warp 1   MMA issuer: one thread issues tcgen05.mma kind::i8 (M=128, N=BLOCK_N, K=32 per
//            instruction), accumulating int32 in TMEM; tcgen05.commit releases the stage and,
//            at the end of a tile, hands the accumulator to the epilogue.
//   warps 2-5 epilogue: tcgen05.ld the accumulator (each thread owns one output row), add bias,
//            ESP-DL's shift/round/saturate with per-channel shifts, ReLU, optional 8-bit LUT,
//            and store NHWC rows with 128-bit writes.  Two TMEM accumulators let the epilogue
//            of tile i overlap the MMAs of tile i+1.
//
// int16 operands: Blackwell tensor cores have no 16-bit integer MMA.  Each operand is split into
// a signed high byte and an unsigned low byte (x = 256*hi + lo); a pre-pass writes the byte planes
// to scratch, and the tile kernel accumulates hi*hi, hi*lo + lo*hi and lo*lo in three TMEM
// accumulators (kind::i8 takes signedness per operand), recombined in 64 bits by the epilogue.
// This is exact as long as K <= 16384 (the partial sums stay below 2^31).
//
// Every mbarrier wait is bounded (about two seconds); on expiry the kernel records
// ESPDL_ERR_TIMEOUT in a device word that espdl_b200_stream_sync reports, and all roles leave.
#include "common.cuh"

#include <cuda.h>

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

namespace {

constexpr int BLOCK_M = 128;
constexpr int NUM_THREADS = 320; // 1 TMA warp + 1 MMA warp + 2 x 4 epilogue warps
constexpr int MAX_STAGES = 12;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

// Per-output-channel epilogue constants staged in shared memory.
struct EpiParams {
    long long bias; // int32 (int8 op) or int64 (int16 op) bias
    int shift;      // out_exponent - filter_exponent[n] - in_exponent, clamped
    int bias_half;  // bias + 2^(shift-1), used by the overflow-free fast form
};

struct TcParams {
    int M, N, K;
    int block_n, n_tiles, m_tiles;
    int swz;          // bytes of K per stage row: 32, 64 or 128
    int k_blocks;     // ceil(K / swz)
    int stages;
    int acc_stages;   // TMEM accumulator buffers (2 for int8, 1 for int16)
    int tmem_cols;    // power of two >= 32
    void *out;
    long long ops;    // output row stride in elements
    const void *bias; // int32[N] or int64[N]
    const int32_t *ew;
    const int8_t *lut;
    int e_shift_base, ew_scalar, per_channel, relu, half_even;
};

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ unsigned long long globaltimer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait on an mbarrier phase.  Returns false when the limit expires.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity)
{
    uint32_t done = 0;
    for (int spin = 0; spin < 64; spin++) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done)
            return true;
    }
    const unsigned long long t0 = globaltimer();
    while (true) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done)
            return true;
        if (globaltimer() - t0 > WAIT_LIMIT_NS)
            return false;
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tc_ld16(uint32_t taddr, int32_t (&v)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// OR-reduction of a predicate over the 128 threads of one epilogue group (named barrier `bar_id`).
__device__ __forceinline__ int __syncthreads_or_group(int pred, int bar_id, int *flag)
{
    if ((threadIdx.x & 127) == 64 % 128 && false)
        *flag = 0;
    // thread 0 of the group clears, everyone ORs, everyone reads
    const int et = (threadIdx.x - 64) & 127;
    if (et == 0)
        *flag = 0;
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
    if (pred)
        atomicOr(flag, 1);
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
    return *flag;
}

// Shared-memory matrix descriptor, K-major operand, swizzled rows of `swz` bytes:
//   bits [0,14)  start address >> 4        bits [16,30) leading byte offset >> 4 (unused here)
//   bits [32,46) stride byte offset >> 4 (distance between 8-row groups = 8 * swz)
//   bits [46,48) descriptor version 1      bits [61,64) swizzle: 2 = 128B, 4 = 64B, 6 = 32B
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, int swz)
{
    const uint64_t layout = swz == 128 ? 2ull : (swz == 64 ? 4ull : 6ull);
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)((8u * (uint32_t)swz) >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= layout << 61;
    return d;
}

// Instruction descriptor of tcgen05.mma kind::i8: D = S32 (bits 4-5 = 2), A/B format at bits 7-9 /
// 10-12 (0 = unsigned 8 bit, 1 = signed 8 bit), both operands K-major, N>>3 at bit 17, M>>4 at bit 24.
__device__ __forceinline__ uint32_t make_idesc(int a_signed, int b_signed, int n)
{
    return (2u << 4) | ((uint32_t)a_signed << 7) | ((uint32_t)b_signed << 10) | ((uint32_t)(n >> 3) << 17) |
        ((uint32_t)(BLOCK_M >> 4) << 24);
}

template <bool I16>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_a_lo, const __grid_constant__ CUtensorMap map_b_lo, const TcParams p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int NPLANE = I16 ? 2 : 1;
    constexpr int NACC = I16 ? 3 : 1;
    const int a_bytes = BLOCK_M * p.swz;
    const int b_bytes = p.block_n * p.swz;
    const int stage_bytes = NPLANE * (a_bytes + b_bytes);
    uint8_t *aux = smem + (size_t)p.stages * stage_bytes;
    // aux: 2 x block_n EpiParams (one set per epilogue group, 16 bytes each), then the barriers
    uint64_t *bars = (uint64_t *)(aux + 2 * sizeof(EpiParams) * p.block_n);
    uint64_t *full_bar = bars, *empty_bar = bars + MAX_STAGES, *tfull_bar = bars + 2 * MAX_STAGES, *tempty_bar = tfull_bar + 2;
    uint32_t *tmem_slot = (uint32_t *)(tempty_bar + 2);
    int *abort_flag = (int *)(tmem_slot + 1);
    int *par_flags = abort_flag + 1; // [2]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = p.m_tiles * p.n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(smem_u32(&tfull_bar[a]), 1);
            mbar_init(smem_u32(&tempty_bar[a]), 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(p.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile / p.n_tiles) * BLOCK_M;
                const int n0 = (tile % p.n_tiles) * p.block_n;
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1)) {
                        ok = false;
                        break;
                    }
                    const uint32_t bar = smem_u32(&full_bar[stage]);
                    uint8_t *st = smem + (size_t)stage * stage_bytes;
                    mbar_arrive_expect_tx(bar, (uint32_t)stage_bytes);
                    tma_load_2d(smem_u32(st), &map_a, kb * p.swz, m0, bar);
                    tma_load_2d(smem_u32(st + NPLANE * a_bytes), &map_b, kb * p.swz, n0, bar);
                    if (I16) {
                        tma_load_2d(smem_u32(st + a_bytes), &map_a_lo, kb * p.swz, m0, bar);
                        tma_load_2d(smem_u32(st + 2 * a_bytes + b_bytes), &map_b_lo, kb * p.swz, n0, bar);
                    }
                    if (++stage == p.stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) {
                atomicExch(&g_tc_error, ESPDL_ERR_TIMEOUT);
                *abort_flag = 1;
            }
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
            const uint32_t idesc_ss = make_idesc(1, 1, p.block_n);
            const uint32_t idesc_su = make_idesc(1, 0, p.block_n);
            const uint32_t idesc_us = make_idesc(0, 1, p.block_n);
            const uint32_t idesc_uu = make_idesc(0, 0, p.block_n);
            const int ksteps = p.swz / 32;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t d0 = tmem_base + (uint32_t)(acc * NACC * p.block_n);
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    if (!mbar_wait(smem_u32(&full_bar[stage]), phase)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t st = smem_u32(smem + (size_t)stage * stage_bytes);
                    const uint64_t da = make_smem_desc(st, p.swz);
                    const uint64_t db = make_smem_desc(st + NPLANE * a_bytes, p.swz);
                    for (int k = 0; k < ksteps; k++) {
                        const uint32_t accum = (kb | k) != 0;
                        const uint64_t koff = (uint64_t)(k * 2); // 32 bytes of K, in 16-byte units
                        if (!I16) {
                            tc_mma_i8(d0, da + koff, db + koff, idesc_ss, accum);
                        } else {
                            const uint64_t da_lo = make_smem_desc(st + a_bytes, p.swz);
                            const uint64_t db_lo = make_smem_desc(st + 2 * a_bytes + b_bytes, p.swz);
                            tc_mma_i8(d0, da + koff, db + koff, idesc_ss, accum);                      // hi * hi
                            tc_mma_i8(d0 + p.block_n, da + koff, db_lo + koff, idesc_su, accum);       // hi * lo
                            tc_mma_i8(d0 + p.block_n, da_lo + koff, db + koff, idesc_us, 1u);          // lo * hi
                            tc_mma_i8(d0 + 2 * p.block_n, da_lo + koff, db_lo + koff, idesc_uu, accum); // lo * lo
                        }
                    }
                    tc_commit(smem_u32(&empty_bar[stage]));
                    if (++stage == p.stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok)
                    break;
                tc_commit(smem_u32(&tfull_bar[acc]));
                if (++acc == p.acc_stages) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
            if (!ok) {
                atomicExch(&g_tc_error, ESPDL_ERR_TIMEOUT);
                *abort_flag = 1;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..9)
        // Two groups of four warps; group g owns TMEM accumulator g and every second tile, so the epilogue of one
        // tile overlaps the accumulator read latency of the other.  (int16: one accumulator set, group 0 only.)
        const int group = (warp - 2) >> 2;
        const int et = (threadIdx.x - 64) & 127;  // thread index inside the group
        const int lane_group = warp & 3;          // TMEM lanes this warp may read: 32*lane_group .. +31
        const int row_in_tile = lane_group * 32 + lane;
        EpiParams *par = (EpiParams *)(aux) + (size_t)group * p.block_n;
        const int acc = group;
        uint32_t acc_phase = 0;
        int loaded_n0 = -1;
        bool fast = false;
        bool ok = true;
        const int bar_id = 1 + group;
        int local = 0;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, local++) {
            if (local % p.acc_stages != group)
                continue;
            const int m0 = (tile / p.n_tiles) * BLOCK_M;
            const int n0 = (tile % p.n_tiles) * p.block_n;
            if (n0 != loaded_n0) {
                // per-channel bias and shift of this N tile (kept across tiles when there is one N tile)
                asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
                int slow = 0;
                for (int j = et; j < p.block_n; j += 128) {
                    const int n = n0 + j;
                    long long b = 0;
                    int sh = 1;
                    if (n < p.N) {
                        if (p.bias)
                            b = I16 ? ((const long long *)p.bias)[n] : (long long)((const int32_t *)p.bias)[n];
                        const int e = p.per_channel ? p.ew[n] : p.ew_scalar;
                        const int lim = I16 ? 62 : 31;
                        sh = max(-lim, min(lim, p.e_shift_base - e));
                    }
                    // Fast form q = (acc + bias + 2^(s-1)) >> s: equal to the reference's wrap-add / 64-bit round as long as
                    // nothing can overflow 32 bits: |acc| <= 2^14 * K < 2^29, |bias| < 2^30, 1 <= s <= 24.
                    if (sh < 1 || sh > 24 || b >= (1ll << 30) || b <= -(1ll << 30))
                        slow = 1;
                    par[j].bias = b;
                    par[j].shift = sh;
                    par[j].bias_half = (int)b + (1 << (max(1, min(24, sh)) - 1));
                }
                const int any_slow = __syncthreads_or_group(slow, bar_id, &par_flags[group]);
                fast = !I16 && !any_slow && !p.half_even && !p.lut && p.K <= 32768;
                loaded_n0 = n0;
            }
            if (!mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase)) {
                ok = false;
                break;
            }
            acc_phase ^= 1;
            tc_fence_after();
            const long long m = (long long)m0 + row_in_tile;
            const uint32_t t0 = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(acc * NACC * p.block_n);
            if (!I16 && fast) {
                int8_t *orow = (int8_t *)p.out + m * p.ops + n0;
                const bool row_ok = m < p.M;
                const bool vec_ok = (p.ops % 16 == 0) && ((((uintptr_t)p.out) + n0) % 16 == 0);
                for (int c0 = 0; c0 < p.block_n; c0 += 32) {
                    const bool two = c0 + 32 <= p.block_n;
                    int32_t v[32];
                    tc_ld16(t0 + c0, *(int32_t(*)[16]) & v[0]);
                    if (two)
                        tc_ld16(t0 + c0 + 16, *(int32_t(*)[16]) & v[16]);
                    tc_ld_wait();
                    uint32_t pk[8];
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        int r[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const EpiParams e = par[c0 + q * 4 + i];
                            int t = (v[q * 4 + i] + e.bias_half) >> e.shift;
                            if (p.relu)
                                t = max(t, 0);
                            r[i] = t;
                        }
                        uint32_t hi, w;
                        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(r[3]), "r"(r[2]));
                        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(r[1]), "r"(r[0]), "r"(hi));
                        pk[q] = w;
                    }
                    if (row_ok) {
                        const int nvalid = p.N - (n0 + c0); // columns of this chunk inside the tensor
                        if (vec_ok && nvalid >= 16) {
                            *(uint4 *)(orow + c0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                            if (two && nvalid >= 32)
                                *(uint4 *)(orow + c0 + 16) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                            else if (two)
                                for (int j = 16; j < 32 && j < nvalid; j++) orow[c0 + j] = (int8_t)(pk[j >> 2] >> (8 * (j & 3)));
                        } else {
                            const int lim = two ? 32 : 16;
                            for (int j = 0; j < lim && j < nvalid; j++) orow[c0 + j] = (int8_t)(pk[j >> 2] >> (8 * (j & 3)));
                        }
                    }
                }
            } else {
                for (int c0 = 0; c0 < p.block_n; c0 += 16) {
                    int32_t v[16];
                    tc_ld16(t0 + c0, v);
                    if (!I16) {
                        tc_ld_wait();
                        if (m < p.M && n0 + c0 < p.N) {
                            uint32_t pk[4];
#pragma unroll
                            for (int q = 0; q < 4; q++) {
                                uint32_t wd = 0;
#pragma unroll
                                for (int i = 0; i < 4; i++) {
                                    const int j = c0 + q * 4 + i;
                                    int32_t r = requant8(v[q * 4 + i], (int32_t)par[j].bias, par[j].shift, p.relu, p.half_even);
                                    if (p.lut)
                                        r = p.lut[(uint8_t)r ^ 0x80u];
                                    wd |= ((uint32_t)r & 0xffu) << (8 * i);
                                }
                                pk[q] = wd;
                            }
                            int8_t *op = (int8_t *)p.out + m * p.ops + n0 + c0;
                            if (n0 + c0 + 16 <= p.N && (((uintptr_t)op) & 15) == 0) {
                                *(uint4 *)op = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                            } else {
                                for (int j = 0; j < 16 && n0 + c0 + j < p.N; j++) op[j] = (int8_t)(pk[j >> 2] >> (8 * (j & 3)));
                            }
                        }
                    } else {
                        int32_t vm[16], vl[16];
                        tc_ld16(t0 + p.block_n + c0, vm);
                        tc_ld16(t0 + 2 * p.block_n + c0, vl);
                        tc_ld_wait();
                        if (m < p.M && n0 + c0 < p.N) {
                            int16_t *op = (int16_t *)p.out + m * p.ops + n0 + c0;
#pragma unroll
                            for (int j = 0; j < 16; j++) {
                                if (n0 + c0 + j < p.N) {
                                    const long long a = ((long long)v[j] << 16) + ((long long)vm[j] << 8) + (long long)vl[j];
                                    op[j] = (int16_t)requant16(a, par[c0 + j].bias, par[c0 + j].shift, p.relu, p.half_even);
                                }
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(smem_u32(&tempty_bar[acc]));
        }
        if (!ok && lane == 0) {
            atomicExch(&g_tc_error, ESPDL_ERR_TIMEOUT);
            *abort_flag = 1;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
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

// 2-D uint8 tensor [rows][cols] with `row_stride` bytes between rows; box = box_rows x box_cols.
int make_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint64_t row_stride, uint32_t box_rows,
             uint32_t box_cols, int swz)
{
    EncodeTiledFn enc = get_encode();
    if (!enc)
        return set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point not found");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {row_stride};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    const CUtensorMapSwizzle sw = swz == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (swz == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
        return ESPDL_ERR_CUDA;
    }
    return ESPDL_OK;
}

int pick_swz(int K)
{
    const int pad32 = (K + 31) / 32 * 32;
    if ((K + 127) / 128 * 128 == pad32)
        return 128;
    if ((K + 63) / 64 * 64 == pad32)
        return 64;
    return 32;
}

constexpr size_t SMEM_BUDGET = 200 * 1024;

bool plan(const espdl_conv_desc &d, TcParams &p)
{
    const bool i16 = d.dtype == ESPDL_DTYPE_INT16;
    const long long M = (long long)d.n * d.out_h * d.out_w;
    if (M > 0x7fffffffll)
        return false;
    p.M = (int)M, p.N = d.out_c, p.K = d.in_c;
    const int max_bn = i16 ? 128 : 256;
    p.n_tiles = (p.N + max_bn - 1) / max_bn;
    p.block_n = (((p.N + p.n_tiles - 1) / p.n_tiles) + 15) / 16 * 16;
    p.n_tiles = (p.N + p.block_n - 1) / p.block_n;
    p.m_tiles = (p.M + BLOCK_M - 1) / BLOCK_M;
    p.swz = pick_swz(p.K);
    p.k_blocks = (p.K + p.swz - 1) / p.swz;
    p.acc_stages = i16 ? 1 : 2;
    int cols = p.acc_stages * (i16 ? 3 : 1) * p.block_n;
    int pow2 = 32;
    while (pow2 < cols) pow2 *= 2;
    if (pow2 > 512)
        return false;
    p.tmem_cols = pow2;
    const size_t stage_bytes = (size_t)(i16 ? 2 : 1) * (BLOCK_M + p.block_n) * p.swz;
    const size_t aux = 2 * sizeof(EpiParams) * (size_t)p.block_n + (2 * MAX_STAGES + 4) * 8 + 32;
    int stages = (int)((SMEM_BUDGET - aux - 1024) / stage_bytes);
    if (stages < 2)
        return false;
    p.stages = stages > MAX_STAGES ? MAX_STAGES : stages;
    return true;
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

int conv2d_tc(const espdl_conv_desc &d, void *workspace, size_t workspace_bytes, cudaStream_t s)
{
    TcParams p;
    if (!plan(d, p))
        return ESPDL_ERR_UNSUPPORTED;
    const bool i16 = d.dtype == ESPDL_DTYPE_INT16;
    const int ips = d.in_pixel_stride ? d.in_pixel_stride : d.in_c;
    p.out = d.output;
    p.ops = d.out_pixel_stride ? d.out_pixel_stride : d.out_c;
    p.bias = d.bias, p.ew = d.filter_exponents, p.lut = d.lut;
    p.e_shift_base = d.out_exponent - d.in_exponent;
    p.ew_scalar = d.filter_exponent, p.per_channel = d.per_channel;
    p.relu = d.activation == ESPDL_ACT_RELU, p.half_even = d.round_mode == ESPDL_ROUND_HALF_EVEN;

    CUtensorMap ma, mb, ma_lo, mb_lo;
    int st;
    if (!i16) {
        if ((st = make_map(&ma, d.input, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)ips, BLOCK_M, (uint32_t)p.swz, p.swz)))
            return st;
        if ((st = make_map(&mb, d.filter, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)p.K, (uint32_t)p.block_n, (uint32_t)p.swz, p.swz)))
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
    size_t smem = 1024 + (size_t)p.stages * stage_bytes + 2 * sizeof(EpiParams) * (size_t)p.block_n + (2 * MAX_STAGES + 4) * 8 + 32;
    if (smem < 120 * 1024) // more than half an SM's shared memory: one CTA per SM, so TMEM allocation never waits on a neighbour
        smem = 120 * 1024;
    const int grid = min(p.m_tiles * p.n_tiles, num_sms());
    static std::once_flag attr_once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(attr_once, [] {
        attr_err = cudaFuncSetAttribute(gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(SMEM_BUDGET + 2048));
        if (attr_err == cudaSuccess)
            attr_err = cudaFuncSetAttribute(gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(SMEM_BUDGET + 2048));
    });
    if (attr_err != cudaSuccess)
        return set_cuda_error(attr_err, "cudaFuncSetAttribute(gemm_tc_kernel)");
    if (i16)
        gemm_tc_kernel<true><<<grid, NUM_THREADS, smem, s>>>(ma, mb, ma_lo, mb_lo, p);
    else
        gemm_tc_kernel<false><<<grid, NUM_THREADS, smem, s>>>(ma, mb, ma_lo, mb_lo, p);
    count_launch();
    return check_launch("gemm_tc");
}

} // namespace espdl
