// C ABI: life cycle, memory and the conv2d dispatcher (include/espdl_b200.h).
#include "common.cuh"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <unordered_map>

namespace espdl {

static thread_local char g_last_error[512] = "";
static std::atomic<uint64_t> g_launches{0};
static int g_device = -1;
static int g_num_sms = 0;
static std::mutex g_ws_mutex;
static void *g_ws = nullptr; // cached scratch of espdl_b200_conv2d (int16 limb planes)
static size_t g_ws_bytes = 0;

int set_cuda_error(cudaError_t e, const char *what)
{
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
    return ESPDL_ERR_CUDA;
}

int set_error_text(int status, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return status;
}

void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

int num_sms() { return g_num_sms > 0 ? g_num_sms : 148; }

namespace {
constexpr int SCHED_PAIRS = 2048;
__device__ unsigned g_sched_words[2 * SCHED_PAIRS]; // zero at load; every kernel leaves its pair zero
}

unsigned *sched_counters(cudaStream_t s)
{
    static std::mutex mu;
    static std::unordered_map<unsigned long long, int> pair_of; // stream handle / capture id -> pair
    static unsigned *base = nullptr;
    static const bool off = getenv("ESPDL_B200_STATIC_TILES") != nullptr;
    if (off)
        return nullptr;
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    unsigned long long id = 0;
    if (cudaStreamGetCaptureInfo(s, &cs, &id) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    // keys: capture ids count up from 1 and stay far below 2^48; stream handles are pointers (or the small legacy values)
    const unsigned long long key = cs == cudaStreamCaptureStatusActive ? (id | (1ull << 63)) : (unsigned long long)(uintptr_t)s;
    std::lock_guard<std::mutex> lock(mu);
    if (!base) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_sched_words) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        base = (unsigned *)p;
    }
    auto it = pair_of.find(key);
    if (it == pair_of.end()) {
        if ((int)pair_of.size() >= SCHED_PAIRS)
            return nullptr;
        it = pair_of.emplace(key, (int)pair_of.size()).first;
    }
    return base + 2 * it->second;
}

int check_launch(const char *what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return set_cuda_error(e, what);
    return ESPDL_OK;
}

} // namespace espdl

using namespace espdl;

extern "C" {

int espdl_b200_init(int device)
{
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        snprintf(g_last_error, sizeof(g_last_error), "no CUDA device: %s", cudaGetErrorString(e));
        return ESPDL_ERR_NO_DEVICE;
    }
    if (device < 0 || device >= count)
        return ESPDL_ERR_INVALID_ARG;
    if (g_device >= 0 && g_device != device)
        // one device per process: the cached scratch and the SM count belong to the device of the first call
        return set_error_text(ESPDL_ERR_INVALID_ARG, "espdl_b200_init(%d): this process is bound to device %d; call espdl_b200_shutdown first",
                              device, g_device);
    ESPDL_CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    ESPDL_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        snprintf(g_last_error, sizeof(g_last_error), "device %d is sm_%d%d; this library holds sm_100a code only", device,
                 prop.major, prop.minor);
        return ESPDL_ERR_NO_DEVICE;
    }
    g_device = device;
    g_num_sms = prop.multiProcessorCount;
    return ESPDL_OK;
}

void espdl_b200_shutdown(void)
{
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    if (g_ws) {
        cudaFree(g_ws);
        g_ws = nullptr;
        g_ws_bytes = 0;
    }
    g_device = -1;
}

const char *espdl_b200_strerror(int status)
{
    switch (status) {
    case ESPDL_OK: return "ok";
    case ESPDL_ERR_INVALID_ARG: return "invalid argument";
    case ESPDL_ERR_UNSUPPORTED: return "unsupported combination";
    case ESPDL_ERR_CUDA: return "CUDA call failed";
    case ESPDL_ERR_NO_DEVICE: return "no usable sm_100 device";
    case ESPDL_ERR_NO_MEM: return "out of device memory";
    case ESPDL_ERR_TIMEOUT: return "device-side wait timed out";
    case ESPDL_ERR_TOO_LARGE: return "size beyond the fixed maximum";
    default: return "unknown status";
    }
}

const char *espdl_b200_last_error(void) { return g_last_error; }

int espdl_b200_arena_alloc(size_t bytes, void **dptr)
{
    if (!dptr)
        return ESPDL_ERR_INVALID_ARG;
    *dptr = nullptr;
    cudaError_t e = cudaMalloc(dptr, bytes ? bytes : 16);
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        return ESPDL_ERR_NO_MEM;
    }
    if (e != cudaSuccess)
        return set_cuda_error(e, "cudaMalloc");
    return ESPDL_OK;
}

int espdl_b200_arena_free(void *dptr)
{
    if (dptr)
        ESPDL_CUDA_TRY(cudaFree(dptr));
    return ESPDL_OK;
}

int espdl_b200_upload(void *dst_dev, const void *src_host, size_t bytes, void *stream)
{
    if ((!dst_dev || !src_host) && bytes)
        return ESPDL_ERR_INVALID_ARG;
    ESPDL_CUDA_TRY(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return ESPDL_OK;
}

int espdl_b200_download(void *dst_host, const void *src_dev, size_t bytes, void *stream)
{
    if ((!dst_host || !src_dev) && bytes)
        return ESPDL_ERR_INVALID_ARG;
    ESPDL_CUDA_TRY(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return ESPDL_OK;
}

} // extern "C"
namespace espdl {
bool pdl_enabled()
{
    static const bool on = !getenv("ESPDL_B200_NO_PDL");
    return on;
}
} // namespace espdl
extern "C" {

int espdl_b200_download_rows(void *dst_host, const void *src_dev, size_t row_bytes, size_t src_stride_bytes, size_t rows, void *stream)
{
    if ((!dst_host || !src_dev) && row_bytes && rows)
        return ESPDL_ERR_INVALID_ARG;
    if (src_stride_bytes < row_bytes)
        return ESPDL_ERR_INVALID_ARG;
    if (!row_bytes || !rows)
        return ESPDL_OK;
    ESPDL_CUDA_TRY(cudaMemcpy2DAsync(dst_host, row_bytes, src_dev, src_stride_bytes, row_bytes, rows, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return ESPDL_OK;
}

int espdl_b200_memset(void *dst_dev, int value, size_t bytes, void *stream)
{
    ESPDL_CUDA_TRY(cudaMemsetAsync(dst_dev, value, bytes, (cudaStream_t)stream));
    return ESPDL_OK;
}

int espdl_b200_stream_sync(void *stream)
{
    ESPDL_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    // a tile kernel whose bounded wait expired leaves its status in a device word
    int dev = read_and_clear_device_error();
    const int dev_stem = read_and_clear_device_error_stem();
    const int dev_dw = read_and_clear_device_error_dw();
    const int dev_conv = read_and_clear_device_error_conv();
    const int dev_block = read_and_clear_device_error_block();
    const int dev_dwpw = read_and_clear_device_error_dwpw();
    const int dev_band = read_and_clear_device_error_band();
    if (!dev)
        dev = dev_stem ? dev_stem : (dev_conv ? dev_conv : (dev_block ? dev_block : (dev_dw ? dev_dw : (dev_dwpw ? dev_dwpw : dev_band))));
    if (dev) {
        snprintf(g_last_error, sizeof(g_last_error), "a device-side bounded wait expired in the tensor-core tile kernel");
        return dev;
    }
    return ESPDL_OK;
}

int espdl_b200_host_alloc(size_t bytes, void **hptr)
{
    if (!hptr)
        return ESPDL_ERR_INVALID_ARG;
    ESPDL_CUDA_TRY(cudaMallocHost(hptr, bytes ? bytes : 16));
    return ESPDL_OK;
}

int espdl_b200_host_free(void *hptr)
{
    if (hptr)
        ESPDL_CUDA_TRY(cudaFreeHost(hptr));
    return ESPDL_OK;
}

uint64_t espdl_b200_launch_count(void) { return g_launches.load(); }

int espdl_b200_mem_info(size_t *free_bytes, size_t *total_bytes)
{
    size_t f = 0, t = 0;
    ESPDL_CUDA_TRY(cudaMemGetInfo(&f, &t));
    if (free_bytes)
        *free_bytes = f;
    if (total_bytes)
        *total_bytes = t;
    return ESPDL_OK;
}

int espdl_b200_stream_create(void **stream)
{
    if (!stream)
        return ESPDL_ERR_INVALID_ARG;
    cudaStream_t s;
    ESPDL_CUDA_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream = (void *)s;
    return ESPDL_OK;
}

int espdl_b200_stream_destroy(void *stream)
{
    if (stream)
        ESPDL_CUDA_TRY(cudaStreamDestroy((cudaStream_t)stream));
    return ESPDL_OK;
}

int espdl_b200_event_create(void **event)
{
    if (!event)
        return ESPDL_ERR_INVALID_ARG;
    cudaEvent_t e;
    ESPDL_CUDA_TRY(cudaEventCreate(&e));
    *event = (void *)e;
    return ESPDL_OK;
}

int espdl_b200_event_destroy(void *event)
{
    if (event)
        ESPDL_CUDA_TRY(cudaEventDestroy((cudaEvent_t)event));
    return ESPDL_OK;
}

int espdl_b200_event_record(void *event, void *stream)
{
    if (!event)
        return ESPDL_ERR_INVALID_ARG;
    ESPDL_CUDA_TRY(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream));
    return ESPDL_OK;
}

int espdl_b200_event_elapsed_ms(void *start, void *stop, float *ms)
{
    if (!start || !stop || !ms)
        return ESPDL_ERR_INVALID_ARG;
    ESPDL_CUDA_TRY(cudaEventSynchronize((cudaEvent_t)stop));
    ESPDL_CUDA_TRY(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    return ESPDL_OK;
}

int espdl_b200_event_sync(void *event)
{
    if (!event)
        return ESPDL_ERR_INVALID_ARG;
    ESPDL_CUDA_TRY(cudaEventSynchronize((cudaEvent_t)event));
    return ESPDL_OK;
}

int espdl_b200_stream_wait_event(void *stream, void *event)
{
    if (!event)
        return ESPDL_ERR_INVALID_ARG;
    ESPDL_CUDA_TRY(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0));
    return ESPDL_OK;
}

int espdl_b200_device_copy(void *dst_dev, const void *src_dev, size_t bytes, void *stream)
{
    if ((!dst_dev || !src_dev) && bytes)
        return ESPDL_ERR_INVALID_ARG;
    ESPDL_CUDA_TRY(cudaMemcpyAsync(dst_dev, src_dev, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return ESPDL_OK;
}

int espdl_b200_graph_begin(void *stream)
{
    if (!stream)
        return ESPDL_ERR_INVALID_ARG; // the legacy default stream cannot be captured
    ESPDL_CUDA_TRY(cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeThreadLocal));
    return ESPDL_OK;
}

int espdl_b200_graph_end(void *stream, void **graph)
{
    if (!stream || !graph)
        return ESPDL_ERR_INVALID_ARG;
    cudaGraph_t g = nullptr;
    ESPDL_CUDA_TRY(cudaStreamEndCapture((cudaStream_t)stream, &g));
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaGraphInstantiate(&exec, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess)
        return set_cuda_error(e, "cudaGraphInstantiate");
    *graph = (void *)exec;
    return ESPDL_OK;
}

int espdl_b200_graph_launch(void *graph, void *stream)
{
    if (!graph)
        return ESPDL_ERR_INVALID_ARG;
    ESPDL_CUDA_TRY(cudaGraphLaunch((cudaGraphExec_t)graph, (cudaStream_t)stream));
    return ESPDL_OK;
}

int espdl_b200_graph_destroy(void *graph)
{
    if (graph)
        ESPDL_CUDA_TRY(cudaGraphExecDestroy((cudaGraphExec_t)graph));
    return ESPDL_OK;
}

} // extern "C"

// ------------------------------------------------------------------ conv2d
// Checks every conv entry point makes before anything is planned or launched: pointers, extents, the output size
// the reference derives, exponent pointers that the kernels will dereference, and the supported enumerators.
int espdl::conv_validate(const espdl_conv_desc *d)
{
    if (!d || !d->input || !d->filter || !d->output)
        return ESPDL_ERR_INVALID_ARG;
    if (d->dtype != ESPDL_DTYPE_INT8 && d->dtype != ESPDL_DTYPE_INT16)
        return ESPDL_ERR_UNSUPPORTED;
    if (d->n < 0 || d->in_h <= 0 || d->in_w <= 0 || d->in_c <= 0 || d->out_c <= 0 || d->out_h <= 0 || d->out_w <= 0)
        return ESPDL_ERR_INVALID_ARG;
    if (d->kh <= 0 || d->kw <= 0 || d->stride_h <= 0 || d->stride_w <= 0 || d->dilation_h <= 0 || d->dilation_w <= 0)
        return ESPDL_ERR_INVALID_ARG;
    if (d->pad_top < 0 || d->pad_bottom < 0 || d->pad_left < 0 || d->pad_right < 0)
        return ESPDL_ERR_INVALID_ARG;
    if (d->group != 1 && !(d->group == d->in_c && d->out_c == d->in_c))
        return ESPDL_ERR_UNSUPPORTED;
    if (d->per_channel && !d->filter_exponents)
        return ESPDL_ERR_INVALID_ARG;
    if (d->activation != ESPDL_ACT_LINEAR && d->activation != ESPDL_ACT_RELU)
        return ESPDL_ERR_UNSUPPORTED;
    if (d->round_mode != ESPDL_ROUND_HALF_UP && d->round_mode != ESPDL_ROUND_HALF_EVEN)
        return ESPDL_ERR_INVALID_ARG;
    if (d->lut && d->dtype != ESPDL_DTYPE_INT8)
        return ESPDL_ERR_UNSUPPORTED;
    if (d->lut_channel_stride != 0 && (!d->lut || d->lut_channel_stride < 256))
        return ESPDL_ERR_INVALID_ARG;
    if ((d->in_pixel_stride && d->in_pixel_stride < d->in_c) || (d->out_pixel_stride && d->out_pixel_stride < d->out_c))
        return ESPDL_ERR_INVALID_ARG;
    if (d->filter_image_stride != 0 && d->group != 1)
        return ESPDL_ERR_INVALID_ARG;
    if (d->residual && (d->dtype != ESPDL_DTYPE_INT8 || d->group != 1 || d->kh != 1 || d->kw != 1 || d->stride_h != 1 || d->stride_w != 1 ||
                        (d->residual_pixel_stride && d->residual_pixel_stride < d->out_c)))
        return ESPDL_ERR_UNSUPPORTED; // the folded Add is implemented for pointwise int8 convs / Gemm
    // output extents must be the ones the reference derives (dl_module_conv.hpp:81-102)
    const int oh = (d->in_h + d->pad_top + d->pad_bottom - d->dilation_h * (d->kh - 1) - 1) / d->stride_h + 1;
    const int ow = (d->in_w + d->pad_left + d->pad_right - d->dilation_w * (d->kw - 1) - 1) / d->stride_w + 1;
    if (oh != d->out_h || ow != d->out_w)
        return ESPDL_ERR_INVALID_ARG;
    if (!d->per_channel) {
        const int shift = d->out_exponent - d->filter_exponent - d->in_exponent;
        const int lim = d->dtype == ESPDL_DTYPE_INT8 ? 31 : 62;
        if (shift > lim || shift < -lim)
            return ESPDL_ERR_INVALID_ARG;
    }
    return ESPDL_OK;
}

extern "C" {

int espdl_b200_conv2d_workspace_bytes(const espdl_conv_desc *desc, size_t *bytes)
{
    if (!bytes)
        return ESPDL_ERR_INVALID_ARG;
    *bytes = 0;
    int st = conv_validate(desc);
    if (st)
        return st;
    if (desc->kernel != ESPDL_KERNEL_SIMT && desc->group == 1 && conv2d_tc_supported(*desc))
        *bytes = conv2d_tc_workspace_bytes(*desc);
    return ESPDL_OK;
}

int espdl_b200_conv2d_ws(const espdl_conv_desc *desc, void *workspace, size_t workspace_bytes, void *stream)
{
    int st = conv_validate(desc);
    if (st)
        return st;
    if (g_device < 0)
        return ESPDL_ERR_NO_DEVICE;
    if (desc->n == 0)
        return ESPDL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (desc->group != 1) {
        // Depthwise convs run on the CUDA cores (dp4a): a tcgen05 MMA of M=128 takes ~143 cycles however small N is,
        // which caps any diagonal-filter formulation on the tensor cores far below the dp4a walk.
        if (desc->kernel == ESPDL_KERNEL_TCGEN05)
            return ESPDL_ERR_UNSUPPORTED;
        // 3x3 int8 with 16-byte channel runs: the TMA-fed kernel; ESPDL_KERNEL_SIMT asks for the kernels that read global
        // memory directly
        if (desc->kernel != ESPDL_KERNEL_SIMT && conv2d_dw_tma_supported(*desc))
            return conv2d_dw_tma(*desc, s);
        return conv2d_depthwise(*desc, s);
    }
    if (desc->kernel != ESPDL_KERNEL_SIMT && conv2d_stem_tc_supported(*desc))
        return conv2d_stem_tc(*desc, s); // 3x3 stride-2 RGB first layer: banded-filter tensor-core kernel
    if (desc->filter_image_stride != 0) {
        // a batch of matrix products: image i multiplies by the filter at filter + i * filter_image_stride
        if (desc->kh != 1 || desc->kw != 1 || desc->stride_h != 1 || desc->stride_w != 1 || desc->pad_top || desc->pad_bottom ||
            desc->pad_left || desc->pad_right || desc->filter_image_stride < 0)
            return ESPDL_ERR_INVALID_ARG;
        if (desc->kernel != ESPDL_KERNEL_SIMT && conv2d_tc_supported(*desc))
            return conv2d_tc(*desc, workspace, workspace_bytes, s);
        if (desc->kernel == ESPDL_KERNEL_TCGEN05)
            return ESPDL_ERR_UNSUPPORTED;
        // 3x3 int8 with 16-byte channel runs: the TMA-fed kernel; ESPDL_KERNEL_SIMT asks for the kernels that read global
        // memory directly
        if (desc->kernel != ESPDL_KERNEL_SIMT && conv2d_dw_tma_supported(*desc))
            return conv2d_dw_tma(*desc, s);
        // shapes the tile kernel does not take: one call per image
        const size_t es = desc->dtype == ESPDL_DTYPE_INT16 ? 2 : 1;
        const long long ips = desc->in_pixel_stride ? desc->in_pixel_stride : desc->in_c;
        const long long ops = desc->out_pixel_stride ? desc->out_pixel_stride : desc->out_c;
        for (int i = 0; i < desc->n; i++) {
            espdl_conv_desc one = *desc;
            one.n = 1, one.filter_image_stride = 0;
            one.input = (const char *)desc->input + (size_t)i * desc->in_h * desc->in_w * ips * es;
            one.filter = (const char *)desc->filter + (size_t)i * desc->filter_image_stride * es;
            one.output = (char *)desc->output + (size_t)i * desc->out_h * desc->out_w * ops * es;
            const int st1 = espdl_b200_conv2d_ws(&one, workspace, workspace_bytes, stream);
            if (st1)
                return st1;
        }
        return ESPDL_OK;
    }
    if (desc->kernel != ESPDL_KERNEL_SIMT && conv2d_band_tc_supported(*desc))
        return conv2d_band_tc(*desc, s); // 3x3 with 8 or 16 input channels: banded filter over 128-byte row windows
    const bool conv_tc_ok = conv2d_conv_tc_supported(*desc);
    if (conv_tc_ok && desc->kernel != ESPDL_KERNEL_SIMT)
        return conv2d_conv_tc(*desc, s); // filters larger than 1x1 (or strided): implicit GEMM over the taps
    const bool tc_ok = conv2d_tc_supported(*desc);
    if (desc->kernel == ESPDL_KERNEL_TCGEN05 && !tc_ok)
        return ESPDL_ERR_UNSUPPORTED;
    if (tc_ok && desc->kernel != ESPDL_KERNEL_SIMT) {
        const size_t need = conv2d_tc_workspace_bytes(*desc);
        if (need > workspace_bytes || (need && !workspace))
            return ESPDL_ERR_INVALID_ARG;
        return conv2d_tc(*desc, workspace, workspace_bytes, s);
    }
    return conv2d_simt(*desc, s);
}

int espdl_b200_conv2d(const espdl_conv_desc *desc, void *stream)
{
    size_t need = 0;
    int st = espdl_b200_conv2d_workspace_bytes(desc, &need);
    if (st)
        return st;
    if (need == 0)
        return espdl_b200_conv2d_ws(desc, nullptr, 0, stream);
    // The cached scratch is shared by all calls of this entry point: calls that need it are
    // serialised on the host here and must be ordered on the device by the caller's streams.
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    if (need > g_ws_bytes) {
        if (g_ws) {
            ESPDL_CUDA_TRY(cudaDeviceSynchronize());
            ESPDL_CUDA_TRY(cudaFree(g_ws));
            g_ws = nullptr;
            g_ws_bytes = 0;
        }
        cudaError_t e = cudaMalloc(&g_ws, need);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return ESPDL_ERR_NO_MEM;
        }
        g_ws_bytes = need;
    }
    return espdl_b200_conv2d_ws(desc, g_ws, g_ws_bytes, stream);
}

int espdl_b200_gemm_scatter(const espdl_conv_desc *desc, void *const *peer_outputs, int n_peers, void *stream)
{
    if (n_peers < 0 || n_peers > 7 || (n_peers > 0 && !peer_outputs))
        return ESPDL_ERR_INVALID_ARG;
    const int st = conv_validate(desc);
    if (st)
        return st;
    if (g_device < 0)
        return ESPDL_ERR_NO_DEVICE;
    if (desc->dtype != ESPDL_DTYPE_INT8 || desc->lut || desc->residual || desc->filter_image_stride != 0 || !conv2d_tc_supported(*desc))
        return ESPDL_ERR_UNSUPPORTED;
    if (desc->n == 0)
        return ESPDL_OK;
    long long delta[7] = {0, 0, 0, 0, 0, 0, 0};
    for (int i = 0; i < n_peers; i++) {
        if (!peer_outputs[i] || ((uintptr_t)peer_outputs[i] % 16) != ((uintptr_t)desc->output % 16))
            return set_error_text(ESPDL_ERR_INVALID_ARG, "espdl_b200_gemm_scatter: peer output %d is null or aligned differently from the local output", i);
        delta[i] = (long long)((intptr_t)peer_outputs[i] - (intptr_t)desc->output);
    }
    return conv2d_tc(*desc, nullptr, 0, (cudaStream_t)stream, delta, n_peers);
}

int espdl_b200_ipc_export(const void *dptr, void *handle64)
{
    if (!dptr || !handle64)
        return ESPDL_ERR_INVALID_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the C ABI passes IPC handles as 64 bytes");
    ESPDL_CUDA_TRY(cudaIpcGetMemHandle((cudaIpcMemHandle_t *)handle64, const_cast<void *>(dptr)));
    return ESPDL_OK;
}

int espdl_b200_ipc_open(const void *handle64, void **dptr)
{
    if (!handle64 || !dptr)
        return ESPDL_ERR_INVALID_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    ESPDL_CUDA_TRY(cudaIpcOpenMemHandle(dptr, h, cudaIpcMemLazyEnablePeerAccess));
    return ESPDL_OK;
}

int espdl_b200_ipc_close(void *dptr)
{
    if (dptr)
        ESPDL_CUDA_TRY(cudaIpcCloseMemHandle(dptr));
    return ESPDL_OK;
}

int espdl_b200_fused_block(const espdl_block_desc *desc, void *stream)
{
    if (!desc)
        return ESPDL_ERR_INVALID_ARG;
    if (!desc->input || !desc->output || !desc->dw_filter || !desc->project_filter || desc->n < 0)
        return ESPDL_ERR_INVALID_ARG;
    if (desc->n == 0)
        return ESPDL_OK;
    // a depthwise -> pointwise pair (no expand conv) has a kernel of its own
    if (!desc->expand_filter && fused_dwpw_supported(*desc, false))
        return fused_dwpw(*desc, (cudaStream_t)stream);
    return fused_block_tc(*desc, (cudaStream_t)stream);
}

int espdl_b200_image_preprocess(const espdl_image_desc *desc, void *stream)
{
    if (!desc)
        return ESPDL_ERR_INVALID_ARG;
    return image_preprocess(*desc, (cudaStream_t)stream);
}

int espdl_b200_detect_candidates(const espdl_detect_desc *desc, void *stream)
{
    if (!desc)
        return ESPDL_ERR_INVALID_ARG;
    return detect_candidates(*desc, (cudaStream_t)stream);
}

int espdl_b200_reduce(const espdl_reduce_desc *desc, void *stream)
{
    if (!desc)
        return ESPDL_ERR_INVALID_ARG;
    return reduce_op(*desc, (cudaStream_t)stream);
}

int espdl_b200_pad(const espdl_pad_desc *desc, void *stream)
{
    if (!desc)
        return ESPDL_ERR_INVALID_ARG;
    return pad_op(*desc, (cudaStream_t)stream);
}

int espdl_b200_fused_block_supported(const espdl_block_desc *desc)
{
    if (!desc)
        return ESPDL_ERR_INVALID_ARG;
    if (desc->reserved[0] == 0 && fused_dwpw_supported(*desc, false))
        return ESPDL_OK;
    return fused_block_supported(*desc) ? ESPDL_OK : ESPDL_ERR_UNSUPPORTED;
}

} // extern "C"
