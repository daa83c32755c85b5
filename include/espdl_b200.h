/*
 * espdl_b200.h - C ABI of the B200 (sm_100a) backend for ESP-DL's quantized
 * operator forward path.
 *
 * ESP-DL itself has no C ABI: its operator layer is a set of C++ free
 * functions that take a pointer to a POD argument block, e.g.
 *   void dl::base::conv2d<int8_t,int32_t,int32_t>(void *args)   esp-dl/dl/base/dl_base_conv2d.hpp:15
 * with args -> dl::base::ArgsType<T>                            esp-dl/dl/base/dl_base.hpp:12-98
 * Each entry point below replaces one family of those functions.  The
 * descriptor structs carry the same information as the reference argument
 * blocks (pointers, NHWC extents, strides/dilations/pads, exponents,
 * activation), but with DEVICE pointers and an explicit batch extent.
 *
 * Conventions
 *  - every function returns ESPDL_OK (0) or a negative ESPDL_ERR_* code and
 *    never throws or aborts;
 *  - kernels are enqueued on the caller's CUDA stream (a cudaStream_t passed
 *    as void*; NULL = the legacy default stream) and are asynchronous;
 *  - all buffers are caller-owned device memory unless stated otherwise;
 *  - activations are NHWC, value = q * 2^exponent (dl::TensorBase,
 *    esp-dl/dl/tensor/include/dl_tensor_base.hpp:297-344);
 *  - convolution filters use the reference's "c" target memory order
 *    [Cout][KH][KW][Cin] (esp-dl/dl/base/dl_base_conv2d.cpp:140-162) and
 *    depthwise filters [KH][KW][C] (esp-dl/dl/base/dl_base_depthwise_conv2d.cpp:47-66).
 */
#ifndef ESPDL_B200_H
#define ESPDL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ status */
#define ESPDL_OK 0
#define ESPDL_ERR_INVALID_ARG (-1) /* NULL pointer, bad extent, bad enum            */
#define ESPDL_ERR_UNSUPPORTED (-2) /* a combination the backend does not implement  */
#define ESPDL_ERR_CUDA (-3)        /* a CUDA runtime/driver call failed             */
#define ESPDL_ERR_NO_DEVICE (-4)   /* no usable sm_100 device / not initialised     */
#define ESPDL_ERR_NO_MEM (-5)      /* device allocation failed                      */
#define ESPDL_ERR_TIMEOUT (-6)     /* a bounded device-side wait expired            */
#define ESPDL_ERR_TOO_LARGE (-7)   /* size beyond a documented fixed maximum        */

/* Same numeric values as dl::dtype_t (esp-dl/dl/tensor/include/dl_tensor_base.hpp:216-233). */
typedef enum {
    ESPDL_DTYPE_FLOAT = 1,
    ESPDL_DTYPE_INT8 = 3,
    ESPDL_DTYPE_INT16 = 5,
    ESPDL_DTYPE_INT32 = 6,
    ESPDL_DTYPE_INT64 = 7,
    ESPDL_DTYPE_BOOL = 9
} espdl_dtype_t;

/* Same numeric values as dl::activation_type_t (esp-dl/dl/dl_define.hpp:108-114). */
typedef enum { ESPDL_ACT_LINEAR = 0, ESPDL_ACT_RELU = 1, ESPDL_ACT_LEAKYRELU = 2, ESPDL_ACT_PRELU = 3 } espdl_act_t;

/* Rounding of the requantisation shift: HALF_UP is what the reference's generic
 * C build does, HALF_EVEN what ESP32-P4 silicon does
 * (esp-dl/dl/dl_define_private.hpp:44-48, esp-dl/dl/tool/src/dl_tool.cpp:95-146). */
typedef enum { ESPDL_ROUND_HALF_UP = 0, ESPDL_ROUND_HALF_EVEN = 1 } espdl_round_t;

/* Kernel selection.  AUTO picks the tensor-core (tcgen05) tile kernel when the
 * shape allows it and the CUDA-core kernel otherwise; the other two values
 * force one path (UNSUPPORTED is returned if it cannot run the shape). */
typedef enum { ESPDL_KERNEL_AUTO = 0, ESPDL_KERNEL_SIMT = 1, ESPDL_KERNEL_TCGEN05 = 2 } espdl_kernel_t;

/* -------------------------------------------------------------- life cycle */
/* Select `device`, check that it is an sm_100 part, create internal state. */
int espdl_b200_init(int device);
void espdl_b200_shutdown(void);
const char *espdl_b200_strerror(int status);
/* Human-readable text of the last failing CUDA call on this thread ("" if none). */
const char *espdl_b200_last_error(void);

/* Device memory for tensors (the arena of dl::ModelContext lives in one such block). */
int espdl_b200_arena_alloc(size_t bytes, void **dptr);
int espdl_b200_arena_free(void *dptr);
int espdl_b200_upload(void *dst_dev, const void *src_host, size_t bytes, void *stream);
int espdl_b200_download(void *dst_host, const void *src_dev, size_t bytes, void *stream);
/* `rows` rows of `row_bytes`, `src_stride_bytes` apart on the device, into a dense host buffer (a tensor that is a
 * channel slice of a wider one). */
int espdl_b200_download_rows(void *dst_host, const void *src_dev, size_t row_bytes, size_t src_stride_bytes, size_t rows, void *stream);
int espdl_b200_memset(void *dst_dev, int value, size_t bytes, void *stream);
int espdl_b200_stream_sync(void *stream);
/* Pinned host staging memory (for the end-to-end path with host buffers). */
int espdl_b200_host_alloc(size_t bytes, void **hptr);
int espdl_b200_host_free(void *hptr);
/* Number of kernels this library has launched since init (all entry points). */
uint64_t espdl_b200_launch_count(void);
/* Free and total bytes of the current device's memory (cudaMemGetInfo): lets a caller check that a region of its
 * program allocated nothing.  Either pointer may be NULL. */
int espdl_b200_mem_info(size_t *free_bytes, size_t *total_bytes);

/* Streams, events and CUDA-graph capture for the layer above (dl::Model runs its plan as one
 * captured graph; dl::Model::profile() times modules with events).  Handles are opaque. */
int espdl_b200_stream_create(void **stream);
int espdl_b200_stream_destroy(void *stream);
int espdl_b200_event_create(void **event);
int espdl_b200_event_destroy(void *event);
int espdl_b200_event_record(void *event, void *stream);
int espdl_b200_event_elapsed_ms(void *start, void *stop, float *ms); /* synchronises on `stop` */
int espdl_b200_event_sync(void *event);                    /* host waits until the event has happened      */
int espdl_b200_stream_wait_event(void *stream, void *event); /* later work on `stream` waits for the event */
int espdl_b200_device_copy(void *dst_dev, const void *src_dev, size_t bytes, void *stream); /* device to device */
int espdl_b200_graph_begin(void *stream);                 /* start capturing work enqueued on `stream`   */
int espdl_b200_graph_end(void *stream, void **graph);     /* stop capturing, instantiate                 */
int espdl_b200_graph_launch(void *graph, void *stream);
int espdl_b200_graph_destroy(void *graph);

/* ------------------------------------------------------------ convolution */
/*
 * Conv2D / pointwise conv / Gemm / MatMul / DepthwiseConv2D, int8 or int16.
 * Replaces dl::base::conv2d<> and dl::base::depthwise_conv2d<>
 * (esp-dl/dl/base/dl_base_conv2d.cpp:1383-1411,912-939;
 *  esp-dl/dl/base/dl_base_depthwise_conv2d.cpp:495,854) including the argument
 * derivation of dl::base::ConvOpArgs (esp-dl/dl/base/dl_base.hpp:132-380).
 *
 *   out[n,y,x,o] = sat( act( rnd( (sum_{ky,kx,c} in[n, y*sh+ky*dh-pt, x*sw+kx*dw-pl, c] * w[o,ky,kx,c]
 *                                  + bias[o]) , shift[o] ) ) )
 *   shift[o] = out_exponent - filter_exponent[o] - in_exponent
 *
 * Taps outside the image are skipped (== zero padding).  A Gemm of A[M,K] by
 * W[N][K] is the call n=1,in_h=1,in_w=M,in_c=K,out_c=N,kh=kw=1
 * (esp-dl/dl/module/include/dl_module_gemm.hpp:85-123).
 * group is 1 (dense) or in_c (depthwise, out_c == in_c).
 */
typedef struct espdl_conv_desc {
    const void *input;                /* NHWC, dtype                                                   */
    const void *filter;               /* [out_c][kh][kw][in_c] (group 1) or [kh][kw][in_c] (depthwise) */
    const void *bias;                 /* int32[out_c] (int8 op) / int64[out_c] (int16 op), or NULL     */
    void *output;                     /* NHWC, dtype                                                   */
    const int32_t *filter_exponents;  /* device int32[out_c] if per_channel, else ignored              */
    const int8_t *lut;                /* optional device int8[256]: out = lut[(uint8)q ^ 0x80] after
                                         the epilogue (a fused dl::module::LUT node); int8 only.  With
                                         lut_channel_stride != 0 one table per output channel:
                                         out = lut[c * lut_channel_stride + ((uint8)q ^ 0x80)]            */
    int32_t dtype;                    /* ESPDL_DTYPE_INT8 or ESPDL_DTYPE_INT16                         */
    int32_t n, in_h, in_w, in_c;
    int32_t out_h, out_w, out_c;
    int32_t kh, kw;
    int32_t stride_h, stride_w;
    int32_t dilation_h, dilation_w;
    int32_t pad_top, pad_bottom, pad_left, pad_right;
    int32_t group;
    int32_t in_pixel_stride;          /* elements between consecutive input pixels; 0 = in_c (dense)   */
    int32_t out_pixel_stride;         /* elements between consecutive output pixels; 0 = out_c (dense);
                                         lets a producer write straight into a Concat slice            */
    int32_t in_exponent, out_exponent;
    int32_t filter_exponent;          /* used when per_channel == 0                                    */
    int32_t per_channel;              /* 0 = per-tensor filter exponent, 1 = filter_exponents[out_c]   */
    int32_t activation;               /* espdl_act_t: LINEAR or RELU                                   */
    int32_t round_mode;               /* espdl_round_t                                                 */
    int32_t kernel;                   /* espdl_kernel_t                                                */
    int32_t filter_image_stride;      /* 0: one filter for all n images (a convolution).  Non-zero: image i uses the
                                         filter at filter + i * filter_image_stride elements - a batch of n
                                         independent matrix products (1x1, group 1 only), which is how MatMul
                                         runs all its slices in one launch                                */
    const void *residual;             /* optional NHWC int8 tensor of the output's shape and exponent that is added
                                         to the result with saturation: out = sat(q + residual), q being the
                                         saturated, activated conv result - a following dl::module::Add with equal
                                         exponents (esp-dl/dl/base/dl_base_add.cpp:8-44) folded into the conv.
                                         int8, group 1, filters without a window only; NULL = none          */
    int32_t residual_pixel_stride;    /* elements between consecutive residual pixels; 0 = out_c (dense)  */
    int32_t lut_channel_stride;       /* 0: `lut` is one table.  Else (>= 256) entries between the tables of consecutive
                                         output channels - a per-channel activation folded into the conv, e.g. a following
                                         dl::module::PRelu (esp-dl/dl/base/dl_base_prelu.cpp:7-21) tabulated per channel  */
} espdl_conv_desc;

int espdl_b200_conv2d(const espdl_conv_desc *desc, void *stream);

/*
 * Scratch the int16 tensor-core path needs (the 8-bit limb planes of both
 * operands).  Returns 0 bytes for shapes that need none.  Pass the buffer with
 * espdl_b200_conv2d_ws; espdl_b200_conv2d allocates and caches one internally.
 */
int espdl_b200_conv2d_workspace_bytes(const espdl_conv_desc *desc, size_t *bytes);
int espdl_b200_conv2d_ws(const espdl_conv_desc *desc, void *workspace, size_t workspace_bytes, void *stream);

/*
 * int16 Gemm / pointwise conv (the shapes espdl_b200_conv2d runs on the tensor cores) for callers that must not
 * allocate device memory.  No counterpart in the reference: ESP-DL's int16 Gemm needs no scratch at all.
 *
 * Who needs it: code that runs where cudaMalloc / cudaFree are off limits - inside a region the host application
 * has fenced against allocation (a real-time control or audio loop, a serving process with a fixed memory budget
 * checked at start-up), or under a memory pool that owns the whole device - and that therefore cannot use
 * espdl_b200_conv2d (it grows a cached scratch buffer on demand) and has no buffer to hand to
 * espdl_b200_conv2d_ws.  The 8-bit limb planes of both operands go into an array that is part of the library
 * image, ESPDL_B200_STATIC_SCRATCH_BYTES large; every GPU that loads the library holds it until the process ends.
 *
 *  - scratch needed is what espdl_b200_conv2d_workspace_bytes reports, 2*(M*K + N*K) bytes rounded up; a larger
 *    problem is rejected with ESPDL_ERR_TOO_LARGE, shapes the tensor-core int16 path does not take (K % 16 != 0,
 *    filters other than 1x1, K > 16384) with ESPDL_ERR_UNSUPPORTED;
 *  - the first call on each device looks up the array's device address (cudaGetSymbolAddress) and keeps it; that
 *    first call also makes the CUDA runtime load the kernels and materialise the array on the device, which the
 *    driver may account as device memory: make one warm-up call per device OUTSIDE the allocation-fenced region and
 *    before any stream capture; from the second call on, free device memory does not change
 *    (tests/test_zz_no_alloc.py reads espdl_b200_mem_info around the calls);
 *  - the call itself runs no cudaMalloc, cudaFree or allocating library routine;
 *  - the descriptor is checked like espdl_b200_conv2d's before anything is launched (ESPDL_ERR_INVALID_ARG for a
 *    per-channel flag without an exponent array, output extents that do not follow from the input's, negative sizes);
 *    a fused table, a residual and per-image filters are not offered here (ESPDL_ERR_UNSUPPORTED);
 *  - all calls share the one array and it keeps the previous call's bytes: every call rewrites the part it reads,
 *    so nothing has to be cleared, but two calls that overlap on the GPU (different streams, no ordering) race.
 */
#define ESPDL_B200_STATIC_SCRATCH_BYTES (16u << 20)
int espdl_b200_gemm_s16_static(const espdl_conv_desc *desc, void *stream);

/* ------------------------------------------------------------ elementwise */
typedef enum {
    ESPDL_ELT_ADD = 0,        /* sat(a + b), numpy broadcasting       esp-dl/dl/base/dl_base_add.cpp:8-44          */
    ESPDL_ELT_MUL = 1,        /* sat(round((a*b) * 2^(ea+eb-eo)))     esp-dl/dl/base/dl_base_mul.cpp:9-46          */
    ESPDL_ELT_REQUANTIZE = 2, /* TensorBase::assign: int<->int, float->int, int->float
                                                                      esp-dl/dl/tensor/src/dl_tensor_base.cpp:223-404 */
    ESPDL_ELT_LUT = 3,        /* out = table[(uint8)in ^ 0x80]        esp-dl/dl/base/dl_base_lut.cpp:10-15         */
    ESPDL_ELT_CLIP = 4,       /* sat(round(clamp(q,lo,hi) * 2^(ei-eo))) esp-dl/dl/module/include/dl_module_clip.hpp:78-90 */
    ESPDL_ELT_RELU = 5,       /* max(q,0) then requantise if exponents differ
                                                                      esp-dl/dl/module/include/dl_module_relu.hpp  */
    ESPDL_ELT_PRELU = 6,      /* q<0 ? sat((q*alpha[c]) >> shift) : q esp-dl/dl/base/dl_base_prelu.cpp:5-19        */
    ESPDL_ELT_SUB = 7,        /* sat(a - b)                           esp-dl/dl/base/dl_base_sub.cpp               */
    ESPDL_ELT_MAX = 8,        /* max(a, b) of the raw integers        esp-dl/dl/base/dl_base_max.cpp:9-50          */
    ESPDL_ELT_MIN = 9,        /* min(a, b) of the raw integers        esp-dl/dl/base/dl_base_min.cpp               */
    ESPDL_ELT_DIV = 10,       /* a == 0 ? 0 : b == 0 ? (a > 0 ? max : min) : sat(round(a * R / b)), R = 2^(ea-eb-eo); the
                                 fp32 order depends on which operand is broadcast along the innermost axis: divisor
                                 broadcast -> a * (R / b), else (a * R) / b  esp-dl/dl/base/dl_base_div.cpp:87-207    */
    ESPDL_ELT_MOD = 11,       /* sat(round(fmodf(a*2^ea, b*2^eb) * 2^-eo)), 0 where b == 0
                                                                      esp-dl/dl/base/dl_base_mod.cpp:9-62          */
    ESPDL_ELT_GREATER = 12,   /* comparisons of the raw integers (exponents are not looked at), one bool byte per
                                 element: out_dtype = ESPDL_DTYPE_BOOL  esp-dl/dl/base/dl_base_greater.cpp:9-44      */
    ESPDL_ELT_GREATER_EQUAL = 13,
    ESPDL_ELT_EQUAL = 14,
    ESPDL_ELT_LESS = 15,
    ESPDL_ELT_LESS_EQUAL = 16,
    ESPDL_ELT_POW = 17        /* sat(round(powf(a*2^ea, b*2^eb) * 2^-eo)); a result that is not a finite int32 (NaN, inf)
                                 becomes the minimum, as the reference's float -> int conversion gives on x86.  int8 with `table`
                                 set reads the 256 x 256 answers the host computed with its own powf (bit-exact); without it,
                                 and for int16, powf runs on the device (within 1 of the reference where powf's last bit decides)
                                 esp-dl/dl/base/dl_base_pow.cpp:9-63 */
} espdl_eltwise_op_t;

typedef struct espdl_eltwise_desc {
    const void *input0;
    const void *input1;       /* ADD/MUL/SUB and MAX..LESS_EQUAL: second operand; LUT: int8[256] table, or for int16 tensors an int16 table of
                                 (65536 >> lut_shift) + 1 entries; PRELU: alpha[c]; else NULL                    */
    void *output;             /* may alias input0 or input1 (the planner runs these ops in place)              */
    int32_t op;               /* espdl_eltwise_op_t                                                            */
    int32_t in_dtype;         /* dtype of input0 (and input1 for the two-operand ops)                          */
    int32_t out_dtype;
    int32_t ndim;             /* 1..4; shapes are right-aligned, every input extent is 1 or the output extent  */
    int32_t out_shape[4];
    int32_t in0_shape[4];
    int32_t in1_shape[4];
    int32_t in0_exponent, in1_exponent, out_exponent;
    int32_t clip_lo, clip_hi; /* CLIP: bounds in the input's quantised scale                                   */
    int32_t round_mode;
    int32_t lut_shift;        /* int16 LUT: log2 of the table step (5 for the usual 2049 entries): index = ((uint16)x ^ 0x8000)
                                 >> lut_shift, rounded to nearest (ties up, or to even with ROUND_HALF_EVEN), esp-dl/dl/base/
                                 dl_base_lut.cpp:50-107; 0 = a full 65536-entry table                             */
    const void *table;        /* POW, int8: int8[256][256], entry [(uint8)a ^ 0x80][(uint8)b ^ 0x80]; else NULL */
    int64_t in0_row_stride;   /* elements between consecutive rows of the innermost axis (a channel slice of a wider     */
    int64_t in1_row_stride;   /* tensor); 0 = dense.  Only for a tensor whose innermost extent equals the output's;     */
    int64_t out_row_stride;   /* not with DIV.  Rows and strides that are multiples of 16 keep the 16-byte kernels.     */
} espdl_eltwise_desc;

int espdl_b200_eltwise(const espdl_eltwise_desc *desc, void *stream);

/* ---------------------------------------------------------------- pooling */
typedef enum { ESPDL_POOL_MAX = 0, ESPDL_POOL_AVG = 1, ESPDL_POOL_GLOBAL_AVG = 2 } espdl_pool_op_t;

/* Replaces dl::base::max_pool2d<> / avg_pool2d<> (esp-dl/dl/base/dl_base_max_pool2d.cpp:9-27,
 * esp-dl/dl/base/dl_base_avg_pool2d.cpp:10-55).  Max ignores padded taps; average is
 * sat(round(sum * ((2^e_in * (1/area)) * 2^-e_out))) in fp32, area = kh*kw. */
typedef struct espdl_pool_desc {
    const void *input;
    void *output;
    int32_t op;
    int32_t dtype;
    int32_t n, in_h, in_w, c;
    int32_t out_h, out_w;
    int32_t kh, kw;
    int32_t stride_h, stride_w;
    int32_t pad_top, pad_bottom, pad_left, pad_right;
    int32_t in_exponent, out_exponent;
} espdl_pool_desc;

int espdl_b200_pool(const espdl_pool_desc *desc, void *stream);

/* ----------------------------------------------------------------- resize */
/* Nearest-neighbour resize (asymmetric / floor), dl::base::resize<>
 * (esp-dl/dl/base/dl_base_resize.cpp:7-35,239-279). */
typedef struct espdl_resize_desc {
    const void *input;
    void *output;
    int32_t dtype;
    int32_t n, in_h, in_w, c;
    int32_t out_h, out_w;
    float scale_h, scale_w;
    int32_t in_exponent, out_exponent;
    int32_t out_pixel_stride; /* 0 = c */
    int32_t mode;             /* 0 nearest (asymmetric, floor); 1 linear with half-pixel coordinates; 2 linear with
                                 align_corners (esp-dl/dl/base/dl_base_resize.cpp:80-236): bilinear for 4-D tensors,
                                 linear along w when in_h == out_h == 1 */
} espdl_resize_desc;

int espdl_b200_resize(const espdl_resize_desc *desc, void *stream);

/* ------------------------------------------------------------------- copy */
/* Strided gather/scatter copy used for Concat / Split / Transpose / Slice
 * (esp-dl/dl/module/include/dl_module_concat.hpp:38-107 and friends):
 * dst[sum i_k*dst_stride[k]] = src[sum i_k*src_stride[k]] for i in shape. */
typedef struct espdl_copy_desc {
    const void *src;
    void *dst;
    int32_t elem_size; /* bytes: 1, 2, 4 or 8 */
    int32_t ndim;      /* 1..6 */
    int32_t shape[6];
    int64_t src_stride[6]; /* in elements */
    int64_t dst_stride[6];
} espdl_copy_desc;

int espdl_b200_copy(const espdl_copy_desc *desc, void *stream);

/* Concat / Split along one axis in ONE launch (esp-dl/dl/module/include/dl_module_concat.hpp:38-107, dl_module_split.hpp):
 * the "wide" tensor is [rows][sum of part_bytes], part i is a dense [rows][part_bytes[i]]; split = 0 gathers the parts
 * into the wide tensor (Concat), split = 1 scatters the wide tensor into the parts (Split).  Every part_bytes[i] and every
 * base address is a multiple of 16: threads move 16-byte units of the wide tensor's rows, so both sides of the copy are
 * whole sectors.  Other shapes go through espdl_b200_copy, one launch per part. */
typedef struct espdl_parts_desc {
    void *wide;
    void *parts[8];
    int64_t part_bytes[8];
    int32_t n_parts; /* 1..8 */
    int32_t split;
    int64_t rows;
    int64_t part_stride[8]; /* bytes between consecutive rows of part i (a multiple of 16); 0 = dense (part_bytes[i]) */
    int32_t skip[8];        /* non-zero: part i is already where it belongs (it lives inside the wide tensor): its
                               columns are left alone and parts[i] is not read                                       */
} espdl_parts_desc;

int espdl_b200_concat_split(const espdl_parts_desc *desc, void *stream);

/* ----------------------------------------------------------------- gather */
/* dl::module::Gather (esp-dl/dl/module/include/dl_module_gather.hpp:66-96): out[o][i][:] = in[o][indices[i]][:] for
 * o < outer, i < num_indices, rows of `inner` elements.  Indices are int32 in device memory and must lie in
 * [0, axis_size): the reference reads whatever an index outside that range points at, this entry point writes
 * nothing for it and returns ESPDL_ERR_INVALID_ARG only for a bad descriptor (the host module checks the values
 * when it loads the node). */
typedef struct espdl_gather_desc {
    const void *input;
    void *output;
    const int32_t *indices; /* device */
    int32_t elem_size;      /* bytes: 1, 2, 4 or 8 */
    int32_t num_indices;
    int64_t outer, axis_size, inner;
} espdl_gather_desc;

int espdl_b200_gather(const espdl_gather_desc *desc, void *stream);

/* ---------------------------------------------------------------- softmax */
/* int8 Softmax along the last axis with the reference's 256-entry exp table
 * (esp-dl/dl/module/include/dl_module_softmax.hpp:148-187): the row sum is a
 * sequential fp32 sum.  out_dtype FLOAT writes y; INT8/INT16 additionally apply
 * the following QuantizeLinear, sat(round(y * 2^-out_exponent)). */
typedef struct espdl_softmax_desc {
    const int8_t *input;
    void *output;
    const float *exp_table; /* device float[256], entry k = expf(2^in_exponent * (k - 128)) */
    int32_t rows, len;       /* rows = outer * inner */
    int32_t out_dtype;
    int32_t out_exponent;
    int32_t inner;           /* elements between neighbours along the softmax axis (0 or 1: the last axis) */
    int32_t log;             /* 1: LogSoftmax, y = 2^in_exponent * x - logf(sum)
                                esp-dl/dl/module/include/dl_module_log_softmax.hpp:150-215 (logf on the device) */
    int32_t in_exponent;     /* LogSoftmax only */
    int32_t round_mode;      /* rounding of the INT8 / INT16 output (the QuantizeLinear that follows, folded in) */
} espdl_softmax_desc;

int espdl_b200_softmax(const espdl_softmax_desc *desc, void *stream);

/* ---------------------------------------------------------- Gemm whose rows also go to other GPUs */
/* N-sharded Gemm without a gather: every rank computes its block of output columns (espdl_conv_desc with the
 * 1x1 / Gemm geometry of dl::module::Gemm, esp-dl/dl/module/include/dl_module_gemm.hpp:85-123; output = its column
 * offset inside the [M][N] result, out_pixel_stride = N) and the kernel's epilogue stores every row into the local
 * result and into the same place of up to seven peers' results (peer-mapped device pointers, plain stores over NVLink).
 * int8 only.  The stores are complete when the kernel is; ranks order their reads behind one another's kernels with
 * whatever they already use between steps (a stream-ordered collective, an event).  K is not split, so no partial
 * sum crosses a GPU and the result equals the one-GPU Gemm bit for bit.
 * espdl_b200_ipc_export / _open / _close hand a buffer of espdl_b200_arena_alloc to another process of the same
 * machine (64-byte handle, cudaIpcMemHandle_t); a pointer returned by _open is valid in calls of this library only
 * as an output of espdl_b200_gemm_scatter or as an operand of espdl_b200_device_copy. */
int espdl_b200_gemm_scatter(const espdl_conv_desc *desc, void *const *peer_outputs, int n_peers, void *stream);
int espdl_b200_ipc_export(const void *dptr, void *handle64);
int espdl_b200_ipc_open(const void *handle64, void **dptr);
int espdl_b200_ipc_close(void *dptr);

/* ---------------------------------------------------------- fused inverted-residual block */
/* One launch for the MobileNetV2 block: 1x1 expand conv -> 3x3 depthwise conv (stride 1 or 2) -> 1x1 project conv
 * (-> residual Add).  In the reference these are three or four nodes, each a dl::module::Conv / Add forward
 * (esp-dl/dl/module/include/dl_module_conv.hpp, dl_module_add.hpp:43-82) over dl::base::conv2d<int8_t,...>,
 * depthwise_conv2d<int8_t,...> and elemwise_add (esp-dl/dl/base/dl_base_conv2d.cpp:9-163,
 * dl_base_depthwise_conv2d.cpp:9-66, dl_base_add.cpp:8-44); every intermediate tensor is requantised to int8
 * exactly as the separate nodes do, it just never leaves the SM.  expand_filter == NULL starts the block at the
 * depthwise conv (hidden_c == in_c), which is the reference's depthwise -> pointwise pair.
 * Returns ESPDL_ERR_UNSUPPORTED for shapes the kernel does not take (int16, in_c or hidden_c not a multiple of 16,
 * a filter other than 3x3, ...): the caller then issues the separate convolutions. */
typedef struct espdl_block_desc {
    const void *input;                      /* [n][in_h][in_w][in_c] int8                                       */
    void *output;                           /* [n][out_h][out_w][out_c] int8                                    */
    const void *expand_filter;              /* [hidden_c][in_c] int8, or NULL                                   */
    const void *expand_bias;                /* int32[hidden_c] or NULL                                          */
    const int32_t *expand_filter_exponents; /* int32[hidden_c] when per_channel bit 0 is set                    */
    const void *dw_filter;                  /* [3][3][hidden_c] int8                                            */
    const void *dw_bias;
    const int32_t *dw_filter_exponents;     /* per_channel bit 1                                                */
    const void *project_filter;             /* [out_c][hidden_c] int8                                           */
    const void *project_bias;
    const int32_t *project_filter_exponents;/* per_channel bit 2                                                */
    const void *residual;                   /* NULL, or a tensor of the output's shape and exponent that is added
                                               with saturation (out = sat(sat(q) + r))                          */
    int32_t dtype;                          /* ESPDL_DTYPE_INT8                                                 */
    int32_t n, in_h, in_w, in_c, hidden_c, out_h, out_w, out_c;
    int32_t stride, pad_top, pad_left;      /* of the depthwise conv; taps outside the image count as zero      */
    int32_t in_exponent, expand_exponent, dw_exponent, out_exponent; /* of the four activation tensors           */
    int32_t expand_filter_exponent, dw_filter_exponent, project_filter_exponent; /* per-tensor filter exponents  */
    int32_t per_channel;
    int32_t expand_activation, dw_activation, project_activation;   /* espdl_act_t: LINEAR or RELU               */
    int32_t expand_clip_max, dw_clip_max;   /* upper clamp of that stage's int8 result: a Clip node of equal
                                               exponents folded in ("ReLU6 via clamp"); 127 = none              */
    int32_t round_mode;
    int32_t reserved[2];
} espdl_block_desc;

int espdl_b200_fused_block(const espdl_block_desc *desc, void *stream);
/* Shape-only question, asked while a graph is planned and no buffer exists yet: ESPDL_OK if espdl_b200_fused_block
 * takes a block of these extents, strides and pads, ESPDL_ERR_UNSUPPORTED otherwise.  Pointers are ignored;
 * reserved[0] != 0 says that the block has an expand conv. */
int espdl_b200_fused_block_supported(const espdl_block_desc *desc);

/* ---------------------------------------------------------- image pre-processing */
/* dl::image::ImagePreprocessor::preprocess (esp-dl/vision/image/dl_image_preprocessor.cpp:106-135) on the device:
 * crop, nearest-neighbour resize (index maps of ImageTransformer::gen_xy_map, esp-dl/vision/image/dl_image_process.cpp:
 * 488-536: source x = min((int)(x * inv_scale_x) + crop_x0, crop_x1 - 1), the same for y, identity when the sizes
 * agree), optional letterbox border, optional R/B swap, and normalise + quantise through a 256-entry table per
 * DESTINATION channel (NormQuant, esp-dl/vision/image/dl_image_norm_quant.hpp:13-49: table[c][v] =
 * quantize((v - mean[c]) * (1/std[c]), 2^-exponent); RGB8882RGB888, dl_image_color_rgb8882rgb888.hpp:51-63).
 * A batch of n images of one size is converted in one launch, straight into the model's input tensor. */
typedef struct espdl_image_desc {
    const uint8_t *input;  /* [n][src_h][src_w][channels] uint8: RGB888 (channels = 3) or GRAY (1)          */
    void *output;          /* [n][dst_h][dst_w][channels] int8 or int16                                     */
    const void *lut;       /* device table [channels][256] of the output type                               */
    int32_t n, src_h, src_w, channels, dst_h, dst_w;
    int32_t out_dtype;     /* ESPDL_DTYPE_INT8 or ESPDL_DTYPE_INT16                                         */
    int32_t crop_x0, crop_y0, crop_x1, crop_y1; /* source area that is resized, x1/y1 exclusive; all 0 = whole image */
    int32_t border_top, border_bottom, border_left, border_right; /* letterbox: destination pixels outside the
                              resized area take the background value                                        */
    int32_t swap_rb;       /* destination channel c reads source channel 2 - c                              */
    uint8_t bg[4];         /* background, in SOURCE channel order                                           */
    float inv_scale_x, inv_scale_y; /* (float)crop_width / inner_dst_width, (float)crop_height / inner_dst_height */
} espdl_image_desc;

int espdl_b200_image_preprocess(const espdl_image_desc *desc, void *stream);

/* ---------------------------------------------------------- detection post-processing: candidate scan */
/* The scan of dl::detect::yolo11PostProcessor::parse_stage (esp-dl/vision/detect/dl_detect_yolo11_postprocessor.cpp:
 * 8-73) over one head: every class score above the quantised threshold becomes a candidate.  The device finds the
 * candidates and packs, per candidate, where it was found, its score code and the box-distribution codes of its
 * pixel; decoding (DFL integral, sigmoid), sorting and NMS are done by the caller with the reference's float
 * arithmetic on these few records.  Records are appended at records[*count ...] (the caller zeroes *count before the
 * first head and may call once per head); the order of the records is not defined, each carries its scan position.
 * int8 tensors. */
typedef struct espdl_detect_record {
    uint16_t image, stage, y, x;
    uint16_t category;
    int8_t score;
    uint8_t pad;
    uint32_t reserved;
    int8_t box[64];            /* the box_channels (<= 64) codes of the pixel                                     */
} espdl_detect_record;

typedef struct espdl_detect_desc {
    const int8_t *score;       /* [n][h][w][classes]                                                              */
    const int8_t *box;         /* [n][h][w][box_channels]                                                         */
    espdl_detect_record *records; /* device array of `capacity` records                                           */
    uint32_t *count;           /* device counter: records found so far (may exceed capacity: then some were dropped) */
    int32_t n, h, w, classes, box_channels;
    int32_t score_threshold;   /* candidates have score code > score_threshold                                    */
    int32_t capacity, stage;
} espdl_detect_desc;

int espdl_b200_detect_candidates(const espdl_detect_desc *desc, void *stream);

/* ---------------------------------------------------------- reductions */
/* ReduceMean / ReduceSum / ReduceMax / ReduceMin over any set of axes (esp-dl/dl/module/include/dl_module_reduce_base.hpp:
 * 121-262 with dl_module_reduce_mean.hpp:17-45, dl_module_reduce_sum.hpp:17-42, dl_module_reduce_max.hpp, _min.hpp).
 * int8 sums in int32, int16 sums in int64.  Mean: round(sum * 2^e_in / count * 2^-e_out) in fp32, in that order;
 * sum: shift_and_round(sum, e_out - e_in); max/min: the code itself.  All saturate to the output type. */
typedef enum {
    ESPDL_REDUCE_MEAN = 0,
    ESPDL_REDUCE_SUM = 1,
    ESPDL_REDUCE_MAX = 2,
    ESPDL_REDUCE_MIN = 3,
    ESPDL_REDUCE_L1 = 4,         /* shift_and_round(sum |x|, e_out - e_in)      esp-dl/dl/module/include/dl_module_reduce_l1.hpp:18-50 */
    ESPDL_REDUCE_SUM_SQUARE = 5, /* shift_and_round(sum x*x, e_out - 2*e_in)    esp-dl/dl/module/include/dl_module_reduce_sum_square.hpp:18-45 */
    ESPDL_REDUCE_L2 = 6,         /* round(sqrt_newton(sum x*x * 2^(2*e_in)) * 2^-e_out), the Newton iteration of
                                    esp-dl/dl/math/include/dl_math.hpp:83-97 in fp32 (at most 100 steps here)
                                    esp-dl/dl/module/include/dl_module_reduce_l2.hpp:17-48 */
    ESPDL_REDUCE_PROD = 7,       /* round(prod(x * 2^e_in) * 2^-e_out): the product runs in element order in fp32 (int8) or
                                    fp64 (int16)      esp-dl/dl/module/include/dl_module_reduce_prod.hpp:18-52 */
    ESPDL_REDUCE_LOG_SUM = 8,    /* round(logf((float)(sum x * 2^e_in)) * 2^-e_out), integer sum
                                    esp-dl/dl/module/include/dl_module_reduce_log_sum.hpp:19-48 */
    ESPDL_REDUCE_LOG_SUM_EXP = 9 /* round(logf(sum exp) * 2^-e_out): fp32 sum in element order of exp_table[x + 128] (int8) or
                                    expf(x * 2^e_in) (int16)   esp-dl/dl/module/include/dl_module_reduce_log_sum_exp.hpp:27-107.
                                    logf / expf run on the device: within 1 of the reference where their last bit decides */
} espdl_reduce_op_t;

typedef struct espdl_reduce_desc {
    const void *input;
    void *output;            /* the kept dims in their order (keepdims only changes the declared shape)  */
    int32_t op, dtype, ndim; /* ndim <= 6                                                                 */
    int32_t shape[6];
    int32_t reduce[6];       /* 1 = this axis is reduced                                                  */
    int32_t in_exponent, out_exponent, round_mode;
    const float *exp_table;  /* LOG_SUM_EXP on int8: device float[256], entry k = expf(2^in_exponent * (k - 128)) */
} espdl_reduce_desc;

int espdl_b200_reduce(const espdl_reduce_desc *desc, void *stream);

/* ---------------------------------------------------------- normalisation */
/* RMSNormalization: dl::module::RMSNormalization::forward_int8 / forward_int16 (esp-dl/dl/module/include/
 * dl_module_rms_normalization.hpp:57-113) with dl::base::rms_norm (esp-dl/dl/base/dl_base_norm.cpp:9-38):
 *   rms = 1 / sqrtf(sum(x*x) * 2^(2*e_in) / len + epsilon) * (2^e_in * 2^-e_out);  y = sat(round((x * rms) * scale[j])),
 * scale float[len].  LayerNormalization: the quantized branch of dl::module::LayerNormalization::forward_template
 * (esp-dl/dl/module/include/dl_module_layer_normalization.hpp:141-214): integer row sum, fp32 variance summed in element
 * order, 1 / sqrt_newton(var + epsilon), y = sat(round((((x*2^e_in - mean) * inv_std) * scale + bias) * 2^-e_out)) with
 * scale / bias of the tensor's integer type (either may be NULL); the optional mean / inv_std_dev outputs hold one
 * value per row.  Rows are the leading axes, len the product of the normalised trailing axes; output may alias input. */
typedef enum { ESPDL_NORM_RMS = 0, ESPDL_NORM_LAYER = 1, ESPDL_NORM_LP = 2 } espdl_norm_op_t;

typedef struct espdl_norm_desc {
    const void *input;
    void *output;
    const void *scale;  /* RMS: float[len]; LAYER: dtype[len] at scale_exponent, or NULL (= 1)                 */
    const void *bias;   /* LAYER: dtype[len] at bias_exponent, or NULL (= 0)                                    */
    void *mean;         /* LAYER: dtype[rows] at mean_exponent, or NULL                                         */
    void *inv_std_dev;  /* LAYER: dtype[rows] at inv_std_dev_exponent, or NULL                                  */
    int32_t op, dtype;  /* espdl_norm_op_t; ESPDL_DTYPE_INT8 or ESPDL_DTYPE_INT16                               */
    int64_t rows;
    int32_t len;
    int32_t in_exponent, out_exponent, scale_exponent, bias_exponent, mean_exponent, inv_std_dev_exponent;
    float epsilon;
    int32_t round_mode;
    int32_t p;          /* LP: 1 or 2.  y = sat(round(x / ||x||_p * 2^-e_out)) along an axis of `len` elements that are `inner`
                           apart (rows = outer * inner); 0 where the norm is 0.  The order of the fp32 operations differs
                           between the last axis and any other, as in the reference
                           esp-dl/dl/module/include/dl_module_lp_normalization.hpp:122-262, 300-356 */
    int64_t inner;      /* LP: 1 = the last axis */
} espdl_norm_desc;

int espdl_b200_norm(const espdl_norm_desc *desc, void *stream);

/* ---------------------------------------------------------- Pad */
/* dl::module::Pad / TensorBase::pad (esp-dl/dl/module/include/dl_module_pad.hpp:10-100, esp-dl/dl/base/dl_base_pad.cpp:
 * 18-66 per axis): constant (the given code), edge (nearest element) or reflect (mirror without repeating the edge). */
typedef enum { ESPDL_PAD_CONSTANT = 0, ESPDL_PAD_EDGE = 1, ESPDL_PAD_REFLECT = 2 } espdl_pad_mode_t;

typedef struct espdl_pad_desc {
    const void *input;
    void *output;
    int32_t elem_size, ndim, mode; /* elem_size 1, 2 or 4 bytes; ndim <= 6 */
    int32_t shape[6];              /* input shape */
    int32_t pad_begin[6], pad_end[6];
    int64_t constant;              /* element value for ESPDL_PAD_CONSTANT (low elem_size bytes) */
} espdl_pad_desc;

int espdl_b200_pad(const espdl_pad_desc *desc, void *stream);

/* ---------------------------------------------------------- ReverseSequence, ScatterND */
/* dl::module::ReverseSequence (esp-dl/dl/module/include/dl_module_reverse_sequence.hpp:14-58): the first two axes are
 * batch and time in either order; for batch b the first seq_lens[b] time steps are reversed, the rest copied. */
typedef struct espdl_reverse_sequence_desc {
    const void *input;
    void *output;            /* not the input buffer */
    const int64_t *seq_lens; /* device int64[batch] */
    int32_t elem_size;       /* 1, 2 or 4 */
    int32_t batch_axis;      /* 0 or 1; the time axis is the other one */
    int32_t dim0, dim1;
    int64_t feature;         /* product of the remaining extents */
} espdl_reverse_sequence_desc;

int espdl_b200_reverse_sequence(const espdl_reverse_sequence_desc *desc, void *stream);

/* dl::module::ScatterND (esp-dl/dl/module/include/dl_module_scatter_nd.hpp:20-228): output = data, then for each of the
 * n_slices index tuples IN ORDER, output[slice] = reduction(output[slice], updates[slice]); add and mul saturate after
 * every step.  Slices addressed twice therefore see the earlier update, as in the reference. */
typedef enum { ESPDL_SCATTER_NONE = 0, ESPDL_SCATTER_ADD = 1, ESPDL_SCATTER_MUL = 2, ESPDL_SCATTER_MAX = 3, ESPDL_SCATTER_MIN = 4 } espdl_scatter_reduction_t;

typedef struct espdl_scatter_nd_desc {
    const void *data;
    const int64_t *indices; /* device int64[n_slices][index_depth] */
    const void *updates;    /* [n_slices][slice_size] */
    void *output;           /* may be the data buffer */
    int32_t dtype;          /* ESPDL_DTYPE_INT8 / INT16 / FLOAT */
    int32_t reduction;      /* espdl_scatter_reduction_t */
    int32_t index_depth;    /* <= 6 */
    int32_t n_slices;
    int64_t slice_size, data_size;
    int64_t axis_offset[6]; /* elements per step of each indexed axis of data */
} espdl_scatter_nd_desc;

int espdl_b200_scatter_nd(const espdl_scatter_nd_desc *desc, void *stream);

/* ---------------------------------------------------------- GRU, LSTM */
/* dl::module::GRU / dl::module::LSTM, quantized (esp-dl/dl/module/include/dl_module_gru.hpp:114-256, dl_module_lstm.hpp:125-300):
 * batch 1, sequence-major X [seq][1][input], W [dir][G*H][input], R [dir][G*H][H], B int16 [dir][2*G*H] at gate_exponent or
 * NULL, initial_h [dir][1][H] or NULL; Y [seq][dir][1][H], Y_h [dir][1][H]; LSTM: initial_c / Y_c int16 [dir][1][H] at
 * gate_exponent.  G = 3 (GRU: z, r, n; linear_before_reset = 1) or 4 (LSTM: i, o, f, c).  The tables are the host's
 * math::SigmoidLUT / math::TanhLUT for gate_exponent: entries 0 .. max (esp-dl/dl/math/include/dl_math.hpp:324-429). */
typedef enum { ESPDL_RNN_GRU = 0, ESPDL_RNN_LSTM = 1 } espdl_rnn_op_t;

typedef struct espdl_rnn_desc {
    const void *x, *w, *r;
    const int16_t *b;
    const void *initial_h;
    const int16_t *initial_c;
    void *y, *y_h;
    int16_t *y_c;
    const float *sigmoid_table, *tanh_table; /* device float[max + 1] */
    int32_t sigmoid_max, tanh_max;
    int32_t op, dtype;                       /* espdl_rnn_op_t; ESPDL_DTYPE_INT8 or ESPDL_DTYPE_INT16 */
    int32_t seq_length, input_size, hidden_size, directions;
    int32_t x_exponent, w_exponent, r_exponent, h_exponent, y_exponent, c_exponent, gate_exponent, round_mode;
} espdl_rnn_desc;

int espdl_b200_rnn(const espdl_rnn_desc *desc, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* ESPDL_B200_H */
