// Building blocks shared by the tensor-core (tcgen05) tile kernels: PTX wrappers for mbarriers, TMA loads,
// tcgen05 MMA / TMEM access, descriptor encoders, and the requantising epilogue that turns one TMEM
// accumulator row (one output pixel, a run of output channels) into saturated int8 and stores it.
#pragma once
#include "common.cuh"

#include <cuda.h>

namespace espdl {
namespace tc {


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

// One probe of an mbarrier phase.  The suspend-time hint lets the hardware park the thread until the phase completes
// (or the hint, in nanoseconds, runs out) instead of returning after the short system default: a waiting warp then
// issues a handful of instructions per hand-over instead of spinning through the issue slots the working warps of its
// scheduler need (a quarter of all instructions of the tile kernels were such spins).
constexpr uint32_t WAIT_HINT_NS = 1000000u;

__device__ __forceinline__ uint32_t mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(WAIT_HINT_NS)
        : "memory");
    return done;
}

// Bounded wait on an mbarrier phase.  Returns false when the limit expires.  The limit is counted on the SM's own
// cycle counter (a read of %globaltimer costs on the order of a microsecond, which a waiter that polls it pays on
// every hand-over of the pipeline); WAIT_LIMIT_CYCLES is about two seconds at the lowest clocks the part runs at.
constexpr long long WAIT_LIMIT_CYCLES = 4000000000ll;

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, long long limit_cycles = WAIT_LIMIT_CYCLES)
{
    if (mbar_try(bar, parity))
        return true;
    const long long t0 = clock64();
    while (true) {
#pragma unroll 1
        for (int spin = 0; spin < 256; spin++) {
            if (mbar_try(bar, parity))
                return true;
            if (limit_cycles < WAIT_LIMIT_CYCLES && clock64() - t0 > limit_cycles) // a short, test-only limit: check every probe
                return false;
        }
        if (clock64() - t0 > limit_cycles)
            return false;
    }
}

__device__ __forceinline__ void fence_barrier_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, int c3, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
        : "memory");
}

// TMA stores (shared -> global), bulk-group completion
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src), "r"(c0), "r"(c1)
                 : "memory");
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2)
{
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map), "r"(src), "r"(c0), "r"(c1),
                 "r"(c2)
                 : "memory");
}

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void named_bar(int id, int nthreads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory"); }

__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Brings a tensor map (a __grid_constant__ kernel parameter) into the descriptor cache ahead of the first copy that uses it.
__device__ __forceinline__ void prefetch_tensormap(const void *map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns: thread t of the warp receives lane (base lane + t), columns c .. c+15.
__device__ __forceinline__ void ld16(uint32_t taddr, int32_t *v)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

// 32 consecutive columns per thread in one instruction.
__device__ __forceinline__ void ld32(uint32_t taddr, int32_t *v)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Waits for the TMEM loads and ties the 16 destination registers to the wait: to the compiler the values only exist
// after this statement, so no arithmetic on them can be scheduled ahead of tcgen05.wait::ld (a tcgen05.ld asm alone
// looks as if it had already produced them).
__device__ __forceinline__ void ld_wait16(int32_t *v)
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]), "+r"(v[9]),
                   "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
                 :
                 : "memory");
}

// Same tie for registers whose load was already waited for by an earlier statement (no instruction is emitted).
__device__ __forceinline__ void tie16(int32_t *v)
{
    asm volatile(""
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]), "+r"(v[9]),
                   "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
                 :
                 : "memory");
}

// Shared-memory matrix descriptor (64 bit):
//   [0,14) start address >> 4   [16,30) leading-dimension byte offset >> 4   [32,46) stride-dimension byte offset >> 4
//   [46,48) version = 1         [61,64) layout: 0 = no swizzle, 2 = 128B, 4 = 64B, 6 = 32B swizzle
// K-major operands.  Swizzled (rows of `swz` bytes): 8-row groups are 8*swz bytes apart (stride offset), the leading
// offset is unused.  Not swizzled: a core matrix is 8 rows x 16 bytes stored contiguously (128 bytes); `lbo` is the
// distance between core matrices that are neighbours along K, `sbo` between neighbours along M/N.
__device__ __forceinline__ uint64_t smem_desc_swizzled(uint32_t addr, int swz)
{
    const uint64_t layout = swz == 128 ? 2ull : (swz == 64 ? 4ull : 6ull);
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)((8u * (uint32_t)swz) >> 4) << 32) | ((uint64_t)1 << 46) |
        (layout << 61);
}

__device__ __forceinline__ uint64_t smem_desc_plain(uint32_t addr, uint32_t lbo, uint32_t sbo)
{
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) |
        ((uint64_t)1 << 46);
}

// Instruction descriptor of tcgen05.mma kind::i8: D = S32 (bits 4-5 = 2), A/B format at bits 7-9 / 10-12
// (0 = unsigned 8 bit, 1 = signed 8 bit), both operands K-major, N>>3 at bit 17, M>>4 at bit 24.
__device__ __forceinline__ uint32_t idesc_i8(int a_signed, int b_signed, int m, int n)
{
    return (2u << 4) | ((uint32_t)a_signed << 7) | ((uint32_t)b_signed << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ------------------------------------------------------------------------------------------ epilogue
// Per-output-channel constants of the fast form, staged in shared memory: q = (acc + bias_half) >> shift with
// bias_half = bias + 2^(shift-1).  Equal to the reference's wrapping 32-bit bias add followed by a 64-bit
// round-half-up shift whenever nothing can overflow 32 bits: |acc| < 2^29, |bias| < 2^30, 1 <= shift <= 24.
struct FastParam {
    int bias_half;
    int shift;
};

struct EpiConfig {
    const void *bias;   // int32[N] (int8 op) / int64[N] (int16 op) or null
    const int32_t *ew;  // per-channel filter exponents or null
    const int8_t *lut;  // optional fused 256-entry table
    int e_shift_base, ew_scalar, per_channel, relu, half_even;
    int lut_stride;     // 0: one table; else entries between the tables of consecutive channels (general epilogue only)
};

// Fills fast[j] for channels [0, n_pad) with `nthreads` cooperating threads (tid in [0, nthreads)).
// Returns 1 in *slow (shared int, pre-zeroed) if any real channel violates the fast form's conditions.
__device__ __forceinline__ void stage_fast_params(const EpiConfig &c, FastParam *fast, int N, int n_pad, int tid, int nthreads, int *slow)
{
    int bad = 0;
    for (int n = tid; n < n_pad; n += nthreads) {
        int b = 0, sh = 1;
        if (n < N) {
            if (c.bias)
                b = ((const int32_t *)c.bias)[n];
            const int e = c.per_channel ? c.ew[n] : c.ew_scalar;
            sh = c.e_shift_base - e;
            if (sh < 1 || sh > 24 || b >= (1 << 30) || b <= -(1 << 30))
                bad = 1;
            sh = max(1, min(24, sh));
        }
        fast[n].bias_half = b + (1 << (sh - 1));
        fast[n].shift = sh;
    }
    if (bad)
        atomicOr(slow, 1);
}

// Requantises 16 accumulator columns with the fast form and packs them to 16 int8 (4 words).
template <bool RELU>
__device__ __forceinline__ void requant16_fast(const int32_t *v, const FastParam *fp, uint32_t *pk)
{
#pragma unroll
    for (int q = 0; q < 4; q++) {
        // two channels per 128-bit shared-memory load
        const int4 p01 = *(const int4 *)(fp + q * 4);
        const int4 p23 = *(const int4 *)(fp + q * 4 + 2);
        const int r0 = (v[q * 4 + 0] + p01.x) >> p01.y;
        const int r1 = (v[q * 4 + 1] + p01.z) >> p01.w;
        const int r2 = (v[q * 4 + 2] + p23.x) >> p23.y;
        const int r3 = (v[q * 4 + 3] + p23.z) >> p23.w;
        uint32_t hi, w;
        if (RELU) {
            // ReLU + saturation: clamp to [0, 255] while packing, then a per-byte minimum with 127
            asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(r3), "r"(r2));
            asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(r1), "r"(r0), "r"(hi));
            w = __vminu4(w, 0x7f7f7f7fu);
        } else {
            asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(r3), "r"(r2));
            asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(r1), "r"(r0), "r"(hi));
        }
        pk[q] = w;
    }
}

// Four accumulator columns -> one word of four saturated int8, constants of the fast form read from shared memory
// (address `fp`, 8 bytes per column) with two 128-bit loads.  With ReLU the add and the lower clamp are one
// instruction (max(acc + bias_half, 0)), which commutes with the arithmetic shift; the pack saturates the top.
// (Volatile loads: letting the compiler hoist them ahead of the TMEM wait cost registers and measured slower.)
template <bool RELU>
__device__ __forceinline__ uint32_t requant4_lean(const int32_t *v, uint32_t fp)
{
    int b0, s0, b1, s1, b2, s2, b3, s3;
    asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(b0), "=r"(s0), "=r"(b1), "=r"(s1) : "r"(fp));
    asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(b2), "=r"(s2), "=r"(b3), "=r"(s3) : "r"(fp + 16));
    int r0, r1, r2, r3;
    if (RELU) {
        r0 = __viaddmax_s32(v[0], b0, 0) >> s0;
        r1 = __viaddmax_s32(v[1], b1, 0) >> s1;
        r2 = __viaddmax_s32(v[2], b2, 0) >> s2;
        r3 = __viaddmax_s32(v[3], b3, 0) >> s3;
    } else {
        r0 = (v[0] + b0) >> s0;
        r1 = (v[1] + b1) >> s1;
        r2 = (v[2] + b2) >> s2;
        r3 = (v[3] + b3) >> s3;
    }
    uint32_t hi, w;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(r3), "r"(r2));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(r1), "r"(r0), "r"(hi));
    return w;
}

// Shared-memory address of the staged constants, produced by a volatile asm: call it AFTER the barrier that follows
// stage_fast_params, so that no load that depends on it can be scheduled before the constants are written.
__device__ __forceinline__ uint32_t epi_param_base(const FastParam *fast)
{
    uint32_t a;
    asm volatile("mov.u32 %0, %1;" : "=r"(a) : "r"(smem_u32(fast)) : "memory");
    return a;
}

template <bool RELU>
__device__ __forceinline__ void requant16_lean(const int32_t *v, uint32_t fp, uint32_t *pk)
{
#pragma unroll
    for (int q = 0; q < 4; q++) pk[q] = requant4_lean<RELU>(v + 4 * q, fp + (uint32_t)(4 * q) * 8u);
}

// One accumulator row (this thread's TMEM lane), columns [0, ncols) of a tile, ncols % 16 == 0, every `parts`-th
// 32-column chunk starting with chunk `part`: requantise with the fast form and store.  `orow` is 16-byte
// aligned; `wide` says it is 32-byte aligned as well (256-bit stores).  TMEM is read 16 columns at a time into
// two register sets in turn: while one half chunk is requantised the load of the next is in flight.
template <bool RELU>
__device__ __forceinline__ void epilogue_lean(uint32_t t0, uint32_t fp, int8_t *orow, int ncols, int parts, int part, bool row_ok, bool wide)
{
    const int step = parts * 32;
    int c0 = part * 32;
    bool have = c0 + 32 <= ncols;
    int32_t va[16], vb[16];
    if (have)
        ld16(t0 + c0, va);
    while (have) {
        uint32_t pk[8];
        ld_wait16(va);
        ld16(t0 + c0 + 16, vb);
        requant16_lean<RELU>(va, fp + (uint32_t)c0 * 8u, pk);
        ld_wait16(vb);
        const int c1 = c0 + step;
        have = c1 + 32 <= ncols;
        if (have)
            ld16(t0 + c1, va);
        requant16_lean<RELU>(vb, fp + (uint32_t)(c0 + 16) * 8u, pk + 4);
        if (row_ok) {
            if (wide) {
                asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(orow + c0), "r"(pk[0]), "r"(pk[1]),
                             "r"(pk[2]), "r"(pk[3]), "r"(pk[4]), "r"(pk[5]), "r"(pk[6]), "r"(pk[7])
                             : "memory");
            } else {
                *(uint4 *)(orow + c0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                *(uint4 *)(orow + c0 + 16) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            }
        }
        c0 = c1;
    }
    if ((ncols & 16) && (ncols >> 5) % parts == part) { // trailing half chunk
        const int ch = ncols - 16;
        int32_t v[16];
        ld16(t0 + ch, v);
        ld_wait16(v);
        uint32_t pk[4];
#pragma unroll
        for (int q = 0; q < 4; q++) pk[q] = requant4_lean<RELU>(v + 4 * q, fp + (uint32_t)(ch + 4 * q) * 8u);
        if (row_ok)
            *(uint4 *)(orow + ch) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
}

// Four accumulator columns -> one word of four saturated int8; `floor_q` is 0 with ReLU and INT_MIN without, so
// the add and the lower clamp are one instruction either way (max commutes with the arithmetic shift).
__device__ __forceinline__ uint32_t requant4_floor(const int32_t *v, uint32_t fp, int floor_q)
{
    int b0, s0, b1, s1, b2, s2, b3, s3;
    asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(b0), "=r"(s0), "=r"(b1), "=r"(s1) : "r"(fp));
    asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(b2), "=r"(s2), "=r"(b3), "=r"(s3) : "r"(fp + 16));
    const int r0 = __viaddmax_s32(v[0], b0, floor_q) >> s0;
    const int r1 = __viaddmax_s32(v[1], b1, floor_q) >> s1;
    const int r2 = __viaddmax_s32(v[2], b2, floor_q) >> s2;
    const int r3 = __viaddmax_s32(v[3], b3, floor_q) >> s3;
    uint32_t hi, w;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(r3), "r"(r2));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(r1), "r"(r0), "r"(hi));
    return w;
}

// Fused 8-bit table (ESP-DL's LUT activations, e.g. Swish: out = table[(uint8)q ^ 0x80], esp-dl/dl/base/dl_base_lut.cpp:10-15)
// for the staged epilogue: the 256 entries sit in shared memory, re-ordered so that the raw output byte is the index
// (entry b holds table[b ^ 0x80]).  Staged once per CTA by `nthreads` cooperating threads.
__device__ __forceinline__ void stage_lut(const int8_t *lut, uint8_t *lut_s, int tid, int nthreads)
{
    for (int i = tid; i < 256; i += nthreads) lut_s[i] = (uint8_t)lut[i ^ 0x80];
}

// Four saturated int8 in a word -> the four table entries: a byte extraction, a one-byte shared-memory load and a
// share of three merges per output.
__device__ __forceinline__ uint32_t lut4(uint32_t w, uint32_t tbl)
{
    const uint32_t i0 = w & 0xffu, i1 = __byte_perm(w, 0u, 0x4441), i2 = __byte_perm(w, 0u, 0x4442), i3 = w >> 24;
    uint32_t b0, b1, b2, b3;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(b0) : "r"(tbl + i0));
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(b1) : "r"(tbl + i1));
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(b2) : "r"(tbl + i2));
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(b3) : "r"(tbl + i3));
    return __byte_perm(__byte_perm(b0, b1, 0x3340), __byte_perm(b2, b3, 0x3340), 0x5410);
}

// Staged epilogue: this thread's accumulator row, PW columns (multiple of 16, at most 128) starting at TMEM address
// t0, requantised and written as row `row` of a [128][PW] byte tile in shared memory, from where one TMA store moves
// the whole tile to global memory in full lines (a thread storing its own row 32 bytes at a time reaches less than
// half of the write bandwidth).  The tile uses the TMA swizzle that matches PW (128-, 64-, 32-byte rows; none for
// other widths): 16-byte chunk index XOR bits 7.. of the byte offset, which for these widths is a function of the
// row alone.  PW is a template parameter so that the walk over the columns is straight-line code; PW = 0 is the
// generic form for any width (`pw`).  TMEM is read 16 columns at a time into two register sets in turn.
template <int PW>
__device__ __forceinline__ void epilogue_stage(uint32_t t0, uint32_t fp, uint32_t buf, int row, int pw, int floor_q)
{
    const int width = PW ? PW : pw;
    uint32_t rx = 0; // what the chunk offset of this row is XORed with
    if (PW == 128)
        rx = ((uint32_t)row & 7u) << 4;
    else if (PW == 64)
        rx = (((uint32_t)row >> 1) & 3u) << 4;
    else if (PW == 32)
        rx = (((uint32_t)row >> 2) & 1u) << 4;
    const uint32_t rb = buf + (uint32_t)(row * width);
    int32_t va[16], vb[16];
    ld16(t0, va);
#pragma unroll
    for (int c = 0; c < (PW ? PW : 128); c += 32) {
        if (!PW && c >= pw)
            break;
        uint32_t pk[4];
        ld_wait16(va);
        const bool second = PW ? (c + 16 < PW) : (c + 16 < pw);
        if (second)
            ld16(t0 + c + 16, vb);
#pragma unroll
        for (int q = 0; q < 4; q++) pk[q] = requant4_floor(va + 4 * q, fp + (uint32_t)(c + 4 * q) * 8u, floor_q);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rb + ((uint32_t)c ^ rx)), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3])
                     : "memory");
        if (!second)
            break;
        ld_wait16(vb);
        const bool more = PW ? (c + 32 < PW) : (c + 32 < pw);
        if (more)
            ld16(t0 + c + 32, va);
#pragma unroll
        for (int q = 0; q < 4; q++) pk[q] = requant4_floor(vb + 4 * q, fp + (uint32_t)(c + 16 + 4 * q) * 8u, floor_q);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rb + ((uint32_t)(c + 16) ^ rx)), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]),
                     "r"(pk[3])
                     : "memory");
    }
}

// Staged epilogue with a fused table: as epilogue_stage, any piece width (a multiple of 16, at most 128; `mask` = 7 / 3 / 0
// is the swizzle of 128- / 64-byte / other rows), every packed word goes through lut4 before it is stored.  A compact
// loop kept out of line: the kernels that call it carry none of its registers in their other epilogues.
static __device__ __noinline__ void epilogue_stage_lut(uint32_t t0, uint32_t fp, uint32_t buf, int row, int pw, uint32_t mask, int floor_q, uint32_t tbl)
{
    const uint32_t rx = ((((uint32_t)(row * pw)) >> 7) & mask) << 4;
    const uint32_t rb = buf + (uint32_t)(row * pw);
#pragma unroll 1
    for (int c = 0; c < pw; c += 16) {
        int32_t v[16];
        uint32_t pk[4];
        ld16(t0 + c, v);
        ld_wait16(v);
#pragma unroll
        for (int q = 0; q < 4; q++) pk[q] = lut4(requant4_floor(v + 4 * q, fp + (uint32_t)(c + 4 * q) * 8u, floor_q), tbl);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rb + ((uint32_t)c ^ rx)), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3])
                     : "memory");
    }
}

// Staged epilogue with a folded Add: as epilogue_stage<0>, and every requantised value is first clamped to int8, then
// summed with the residual byte of the same row and column and saturated again (out = sat(sat(q) + r)).  `res` is
// this thread's residual row at the piece's first column (16-byte aligned); `valid` = columns of the piece inside N.
__device__ __forceinline__ void epilogue_stage_residual(uint32_t t0, uint32_t fp, uint32_t buf, int row, int pw, uint32_t mask, int floor_q,
                                                        const int8_t *res, bool row_ok, int valid)
{
    const uint32_t rbase = (uint32_t)(row * pw);
    for (int c = 0; c < pw; c += 16) {
        int32_t v[16];
        ld16(t0 + c, v);
        ld_wait16(v);
        uint4 rr = make_uint4(0u, 0u, 0u, 0u);
        if (row_ok && c + 16 <= valid)
            rr = __ldg((const uint4 *)(res + c));
        else if (row_ok)
            for (int j = 0; j < 16; j++)
                if (c + j < valid)
                    ((uint8_t *)&rr)[j] = (uint8_t)res[c + j];
        const uint32_t rw[4] = {rr.x, rr.y, rr.z, rr.w};
        uint32_t pk[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            int b[4], s[4];
            asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(b[0]), "=r"(s[0]), "=r"(b[1]), "=r"(s[1]) : "r"(fp + (uint32_t)(c + 4 * q) * 8u));
            asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(b[2]), "=r"(s[2]), "=r"(b[3]), "=r"(s[3]) : "r"(fp + (uint32_t)(c + 4 * q) * 8u + 16u));
            int t[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int qv = min(max(__viaddmax_s32(v[4 * q + i], b[i], floor_q) >> s[i], -128), 127);
                t[i] = qv + (int)(int8_t)(rw[q] >> (8 * i));
            }
            uint32_t hi;
            asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(t[3]), "r"(t[2]));
            asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(pk[q]) : "r"(t[1]), "r"(t[0]), "r"(hi));
        }
        uint32_t off = rbase + (uint32_t)c;
        off ^= ((off >> 7) & mask) << 4;
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(buf + off), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]) : "memory");
    }
}

// General form (any rounding mode, any shift, optional LUT), constants read from global memory.
__device__ __forceinline__ void requant16_general(const int32_t *v, const EpiConfig &c, int n_first, int N, uint32_t *pk)
{
#pragma unroll
    for (int q = 0; q < 4; q++) {
        uint32_t wd = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int n = min(n_first + q * 4 + i, N - 1);
            const int e = c.per_channel ? __ldg(c.ew + n) : c.ew_scalar;
            const int shift = max(-31, min(31, c.e_shift_base - e));
            const int b = c.bias ? __ldg((const int32_t *)c.bias + n) : 0;
            int32_t r = requant8(v[q * 4 + i], b, shift, c.relu, c.half_even);
            if (c.lut)
                r = c.lut[(long long)n * c.lut_stride + ((uint8_t)r ^ 0x80u)];
            wd |= ((uint32_t)r & 0xffu) << (8 * i);
        }
        pk[q] = wd;
    }
}

// Stores `count` (<= 32) packed int8 starting at `dst`; `words` holds them little-endian.  `align` is what the
// caller knows about dst: 16 (16-byte aligned), 8, 4 or 1; the widest stores that alignment allows are used and
// the ragged tail goes out byte by byte.
__device__ __forceinline__ void store_bytes(int8_t *dst, const uint32_t *words, int count, int align)
{
    if (count >= 32 && align >= 16 && (((uintptr_t)dst) & 31) == 0) {
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(words[0]), "r"(words[1]), "r"(words[2]),
                     "r"(words[3]), "r"(words[4]), "r"(words[5]), "r"(words[6]), "r"(words[7])
                     : "memory");
        return;
    }
    int done = 0;
    if (align >= 16) {
        if (count >= 16)
            *(uint4 *)dst = make_uint4(words[0], words[1], words[2], words[3]);
        if (count >= 32)
            *(uint4 *)(dst + 16) = make_uint4(words[4], words[5], words[6], words[7]);
        done = count >= 32 ? 32 : (count >= 16 ? 16 : 0);
    } else if (align >= 8) {
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (8 * j + 8 <= count) {
                *(uint2 *)(dst + 8 * j) = make_uint2(words[2 * j], words[2 * j + 1]);
                done = 8 * j + 8;
            }
    } else if (align >= 4) {
#pragma unroll
        for (int j = 0; j < 8; j++)
            if (4 * j + 4 <= count) {
                *(uint32_t *)(dst + 4 * j) = words[j];
                done = 4 * j + 4;
            }
    }
#pragma unroll
    for (int j = 0; j < 32; j++) // unrolled with static indices so that `words` stays in registers
        if (j >= done && j < count)
            dst[j] = (int8_t)(words[j >> 2] >> (8 * (j & 3)));
}

} // namespace tc
} // namespace espdl
