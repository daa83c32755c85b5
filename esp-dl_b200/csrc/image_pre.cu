// Image pre-processing on the device: crop, nearest-neighbour resize, letterbox border, R/B swap and the
// normalise-and-quantise table, for a batch of images, written straight into the model's NHWC input tensor.
// Replaces dl::image::ImagePreprocessor::preprocess (esp-dl/vision/image/dl_image_preprocessor.cpp:106-135) and the
// nearest-neighbour path of ImageTransformer::transform (esp-dl/vision/image/dl_image_process.cpp:488-536).
// Bandwidth bound: a thread produces one destination pixel (all channels); source rows are read through the
// read-only path, the tables (at most 3 x 256 entries) live in shared memory.
#include "common.cuh"

namespace espdl {

namespace {

struct ImgParams {
    const uint8_t *in;
    void *out;
    const void *lut;
    int n, sh, sw, ch, dh, dw;
    int x0, y0, x1, y1;
    int bt, bb, bl, br;
    int swap, same_size;
    uint8_t bg[4];
    float isx, isy;
    long long total;
};

template <typename T>
__global__ void __launch_bounds__(256) image_pre_kernel(ImgParams p)
{
    __shared__ T lut_s[3 * 256];
    for (int i = threadIdx.x; i < p.ch * 256; i += blockDim.x) lut_s[i] = ((const T *)p.lut)[i];
    __syncthreads();
    const int inner_w = p.dw - p.bl - p.br, inner_h = p.dh - p.bt - p.bb;
    T *out = (T *)p.out;
    for (long long item = blockIdx.x * (long long)blockDim.x + threadIdx.x; item < p.total; item += (long long)gridDim.x * blockDim.x) {
        const int x = (int)(item % p.dw);
        const int y = (int)((item / p.dw) % p.dh);
        const int img = (int)(item / ((long long)p.dw * p.dh));
        const int xi = x - p.bl, yi = y - p.bt;
        uint8_t v[3];
        if (xi < 0 || xi >= inner_w || yi < 0 || yi >= inner_h) {
            for (int c = 0; c < p.ch; c++) v[c] = p.bg[c];
        } else {
            // the reference's index maps: (int)(i * inv_scale) in float, offset by the crop origin, clamped to the crop
            const int sx = p.same_size ? xi + p.x0 : min((int)__fmul_rn((float)xi, p.isx) + p.x0, p.x1 - 1);
            const int sy = p.same_size ? yi + p.y0 : min((int)__fmul_rn((float)yi, p.isy) + p.y0, p.y1 - 1);
            const uint8_t *src = p.in + (((long long)img * p.sh + sy) * p.sw + sx) * p.ch;
            for (int c = 0; c < p.ch; c++) v[c] = __ldg(src + c);
        }
        T *dst = out + item * p.ch;
        if (p.ch == 3) {
            dst[0] = lut_s[v[p.swap ? 2 : 0]];
            dst[1] = lut_s[256 + v[1]];
            dst[2] = lut_s[512 + v[p.swap ? 0 : 2]];
        } else {
            dst[0] = lut_s[v[0]];
        }
    }
}

} // namespace

int image_preprocess(const espdl_image_desc &d, cudaStream_t s)
{
    if (!d.input || !d.output || !d.lut || d.n <= 0 || d.src_h <= 0 || d.src_w <= 0 || d.dst_h <= 0 || d.dst_w <= 0)
        return ESPDL_ERR_INVALID_ARG;
    if ((d.channels != 1 && d.channels != 3) || (d.out_dtype != ESPDL_DTYPE_INT8 && d.out_dtype != ESPDL_DTYPE_INT16))
        return ESPDL_ERR_UNSUPPORTED;
    ImgParams p;
    p.in = d.input, p.out = d.output, p.lut = d.lut;
    p.n = d.n, p.sh = d.src_h, p.sw = d.src_w, p.ch = d.channels, p.dh = d.dst_h, p.dw = d.dst_w;
    const bool whole = d.crop_x0 == 0 && d.crop_y0 == 0 && d.crop_x1 == 0 && d.crop_y1 == 0;
    p.x0 = whole ? 0 : d.crop_x0, p.y0 = whole ? 0 : d.crop_y0, p.x1 = whole ? d.src_w : d.crop_x1, p.y1 = whole ? d.src_h : d.crop_y1;
    if (p.x0 < 0 || p.y0 < 0 || p.x0 >= p.x1 || p.y0 >= p.y1 || p.x1 > d.src_w || p.y1 > d.src_h)
        return ESPDL_ERR_INVALID_ARG;
    p.bt = d.border_top, p.bb = d.border_bottom, p.bl = d.border_left, p.br = d.border_right;
    if (p.bt < 0 || p.bb < 0 || p.bl < 0 || p.br < 0 || p.bt + p.bb > d.dst_h - 1 || p.bl + p.br > d.dst_w - 1)
        return ESPDL_ERR_INVALID_ARG; // dl_image_process.cpp:358-361
    p.swap = d.swap_rb != 0 && d.channels == 3;
    p.same_size = (p.x1 - p.x0) == (d.dst_w - p.bl - p.br) && (p.y1 - p.y0) == (d.dst_h - p.bt - p.bb);
    for (int i = 0; i < 4; i++) p.bg[i] = d.bg[i];
    p.isx = d.inv_scale_x, p.isy = d.inv_scale_y;
    p.total = (long long)d.n * d.dst_h * d.dst_w;
    const long long blocks = (p.total + 255) / 256;
    const int grid = (int)(blocks < (long long)num_sms() * 16 ? blocks : (long long)num_sms() * 16);
    if (d.out_dtype == ESPDL_DTYPE_INT8)
        image_pre_kernel<int8_t><<<grid, 256, 0, s>>>(p);
    else
        image_pre_kernel<int16_t><<<grid, 256, 0, s>>>(p);
    count_launch();
    return check_launch("image_pre");
}

} // namespace espdl
