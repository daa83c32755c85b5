// Shared device/host helpers of the B200 backend: ESP-DL's exact rounding and
// saturation rules as device functions, status plumbing and launch accounting.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/espdl_b200.h"

namespace espdl {

// ---------------------------------------------------------------- host state
int set_cuda_error(cudaError_t e, const char *what); // records text, returns ESPDL_ERR_CUDA
int set_error_text(int status, const char *fmt, ...); // records text for espdl_b200_last_error, returns status
void count_launch(int n = 1);
int num_sms();
// Work counters of a persistent kernel that hands out its tiles dynamically: two zero-initialised words {next tile,
// CTAs done} in device memory that no other launch in flight uses - one pair per stream, or per capture sequence while
// `s` is being captured into a graph (launches of one stream, and the nodes of one graph, run one after the other; two
// graphs may run side by side).  The kernel's last CTA writes both words back to zero.  Null when no pair is left: the
// kernel then walks its tiles in the fixed order.
unsigned *sched_counters(cudaStream_t s);
int lp_norm_op(const espdl_norm_desc &d, cudaStream_t s); // sequence_ops.cu
// Records the most recent failed launch (cudaGetLastError) if any.
int check_launch(const char *what);
// Programmatic dependent launch: the kernel may become resident while the previous kernel of the stream is still
// draining (its CTAs take an SM as soon as one is free and run their prologue: barriers, TMEM, per-channel constants).
// Such a kernel calls grid_dep_wait() before it reads or writes anything a previous kernel touches, and
// grid_dep_launch() once its own CTA is set up.  ESPDL_B200_NO_PDL=1 launches them the plain way.
bool pdl_enabled();

template <typename... KArgs, typename... Args>
cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args &&...args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#ifdef __CUDACC__
// Blocks until every kernel this one depends on has finished and its writes are visible to this grid.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// This CTA no longer minds the next kernel's CTAs becoming resident.
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

#define ESPDL_CUDA_TRY(call)                                \
    do {                                                    \
        cudaError_t e__ = (call);                           \
        if (e__ != cudaSuccess)                             \
            return ::espdl::set_cuda_error(e__, #call);     \
    } while (0)

// Descriptor checks shared by every conv entry point (abi.cu); ESPDL_OK or the status to return.
int conv_validate(const espdl_conv_desc *d);

// kernels behind the C ABI (one translation unit each)
int conv2d_simt(const espdl_conv_desc &d, cudaStream_t s);
int conv2d_depthwise(const espdl_conv_desc &d, cudaStream_t s);
bool conv2d_tc_supported(const espdl_conv_desc &d);
size_t conv2d_tc_workspace_bytes(const espdl_conv_desc &d);
int conv2d_tc(const espdl_conv_desc &d, void *workspace, size_t workspace_bytes, cudaStream_t s, const long long *peer_delta = nullptr,
              int n_peer = 0); // peer_delta: byte distances to copies of the output on other GPUs that receive every row as well
int read_and_clear_device_error(); // status word written by device-side bounded waits (0 = none)
int read_and_clear_device_error_stem();
int read_and_clear_device_error_band();
int read_and_clear_device_error_dw();
int read_and_clear_device_error_conv();
int read_and_clear_device_error_block();
int read_and_clear_device_error_dwpw();
int image_preprocess(const espdl_image_desc &d, cudaStream_t s);
int detect_candidates(const espdl_detect_desc &d, cudaStream_t s);
int reduce_op(const espdl_reduce_desc &d, cudaStream_t s);
int pad_op(const espdl_pad_desc &d, cudaStream_t s);
bool fused_block_supported(const espdl_block_desc &d);
int fused_block_tc(const espdl_block_desc &d, cudaStream_t s);
bool fused_dwpw_supported(const espdl_block_desc &d, bool has_expand); // depthwise -> pointwise pair without an expand conv
int fused_dwpw(const espdl_block_desc &d, cudaStream_t s);
bool conv2d_conv_tc_supported(const espdl_conv_desc &d);
int conv2d_conv_tc(const espdl_conv_desc &d, cudaStream_t s);
bool conv2d_dw_tma_supported(const espdl_conv_desc &d);
int conv2d_dw_tma(const espdl_conv_desc &d, cudaStream_t s);
bool conv2d_stem_tc_supported(const espdl_conv_desc &d);
int conv2d_stem_tc(const espdl_conv_desc &d, cudaStream_t s);
// 3x3 conv with 8 or 16 input channels: banded-filter tensor-core kernel over 128-byte row windows (conv_band_tc.cu)
bool conv2d_band_tc_supported(const espdl_conv_desc &d);
int conv2d_band_tc(const espdl_conv_desc &d, cudaStream_t s);

// ------------------------------------------------------------- device math
// dl::tool::shift_and_round on a 32-bit accumulator (int8 operators).
//   shift > 0 : HALF_UP   floor((v + 2^(s-1)) / 2^s)  ==  (v >> s) + bit (s-1) of v
//               HALF_EVEN floor, +1 if remainder > half or (== half and quotient odd)
//   shift <= 0: (int64)v << -shift, saturated to int32
// Callers guarantee |shift| <= 31.
__device__ __forceinline__ int32_t shift_round32(int32_t v, int shift, int half_even)
{
    if (shift > 0) {
        int32_t q = v >> shift;
        if (!half_even) {
            q += (v >> (shift - 1)) & 1;
        } else {
            const int32_t rem = v & ((1 << shift) - 1);
            const int32_t half = 1 << (shift - 1);
            q += (rem > half || (rem == half && (q & 1))) ? 1 : 0;
        }
        return q;
    }
    const long long s = (long long)v << (-shift);
    return (int32_t)max(min(s, (long long)INT32_MAX), (long long)INT32_MIN);
}

// Same on a 64-bit accumulator (int16 operators); |shift| <= 62.
__device__ __forceinline__ long long shift_round64(long long v, int shift, int half_even)
{
    if (shift > 0) {
        long long q = v >> shift;
        if (!half_even) {
            q += (v >> (shift - 1)) & 1;
        } else {
            const long long rem = v & ((1ll << shift) - 1);
            const long long half = 1ll << (shift - 1);
            q += (rem > half || (rem == half && (q & 1))) ? 1 : 0;
        }
        return q;
    }
    return (long long)((unsigned long long)v << (-shift));
}

__device__ __forceinline__ int32_t sat8(int32_t v) { return max(-128, min(127, v)); }
__device__ __forceinline__ int32_t sat16(int32_t v) { return max(-32768, min(32767, v)); }
__device__ __forceinline__ long long sat16_64(long long v) { return max(-32768ll, min(32767ll, v)); }

// int8 conv epilogue: bias (wrapping 32-bit add), shift/round, ReLU, saturate.
__device__ __forceinline__ int32_t requant8(int32_t acc, int32_t bias, int shift, int relu, int half_even)
{
    int32_t v = shift_round32((int32_t)((uint32_t)acc + (uint32_t)bias), shift, half_even);
    if (relu)
        v = max(v, 0);
    return sat8(v);
}

__device__ __forceinline__ int32_t requant16(long long acc, long long bias, int shift, int relu, int half_even)
{
    long long v = shift_round64(acc + bias, shift, half_even);
    if (relu)
        v = max(v, 0ll);
    return (int32_t)sat16_64(v);
}

// dl::tool::round(float) on generic targets: (int)floorf((float)((double)v + 0.5)).
// A single correctly rounded fp32 add gives the same float as the double sum
// narrowed to float (the double sum of two floats whose exponents differ by less
// than 29 is exact), so one __fadd_rn reproduces it without fp64.
__device__ __forceinline__ int fround_half_up(float v) { return (int)floorf(__fadd_rn(v, 0.5f)); }
// ESP32-P4: fcvt.w.s with round-to-nearest-even.
__device__ __forceinline__ int fround_half_even(float v) { return __float2int_rn(v); }
__device__ __forceinline__ int fround(float v, int half_even) { return half_even ? fround_half_even(v) : fround_half_up(v); }

// DL_SCALE / DL_RESCALE: exact powers of two as floats.
__host__ __device__ __forceinline__ float dl_scale(int e) { return e > 0 ? (float)(1 << e) : 1.0f / (float)(1 << -e); }
__host__ __device__ __forceinline__ float dl_rescale(int e) { return e > 0 ? 1.0f / (float)(1 << e) : (float)(1 << -e); }

} // namespace espdl
