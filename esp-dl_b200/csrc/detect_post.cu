// Candidate scan of the detection post-processor: the O(H*W*classes) part of
// dl::detect::yolo11PostProcessor::parse_stage (esp-dl/vision/detect/dl_detect_yolo11_postprocessor.cpp:8-73) on the
// device.  A thread compares the class scores of one pixel with the quantised threshold (integer compare, as the
// reference) and appends a record per hit; the few records are decoded, sorted and suppressed by the host class
// with the reference's float arithmetic.  Bandwidth bound: the score tensor is read once, 16 bytes at a time.
#include "common.cuh"

namespace espdl {

namespace {

__global__ void __launch_bounds__(256) detect_candidates_kernel(espdl_detect_desc d, long long pixels)
{
    for (long long pix = blockIdx.x * (long long)blockDim.x + threadIdx.x; pix < pixels; pix += (long long)gridDim.x * blockDim.x) {
        const int8_t *sp = d.score + pix * d.classes;
        const bool vec = (d.classes % 16 == 0) && (((uintptr_t)d.score) % 16 == 0);
        for (int c0 = 0; c0 < d.classes; c0 += 16) {
            int8_t v[16];
            const int cnt = min(16, d.classes - c0);
            if (vec) {
                *(uint4 *)v = __ldg((const uint4 *)(sp + c0));
            } else {
                for (int j = 0; j < cnt; j++) v[j] = sp[c0 + j];
            }
            for (int j = 0; j < cnt; j++) {
                if ((int)v[j] <= d.score_threshold)
                    continue;
                const uint32_t slot = atomicAdd(d.count, 1u);
                if (slot >= (uint32_t)d.capacity)
                    continue; // counted, not stored: the caller sees count > capacity
                espdl_detect_record *r = d.records + slot;
                const int x = (int)(pix % d.w), y = (int)((pix / d.w) % d.h), img = (int)(pix / ((long long)d.w * d.h));
                r->image = (uint16_t)img, r->stage = (uint16_t)d.stage, r->y = (uint16_t)y, r->x = (uint16_t)x;
                r->category = (uint16_t)(c0 + j), r->score = v[j], r->pad = 0, r->reserved = 0;
                const int8_t *bp = d.box + pix * d.box_channels;
                for (int k = 0; k < 64; k++) r->box[k] = k < d.box_channels ? bp[k] : (int8_t)0;
            }
        }
    }
}

} // namespace

int detect_candidates(const espdl_detect_desc &d, cudaStream_t s)
{
    if (!d.score || !d.box || !d.records || !d.count || d.n <= 0 || d.h <= 0 || d.w <= 0 || d.classes <= 0 || d.capacity <= 0)
        return ESPDL_ERR_INVALID_ARG;
    if (d.box_channels <= 0 || d.box_channels > 64 || d.n > 65535 || d.h > 65535 || d.w > 65535 || d.classes > 65535)
        return ESPDL_ERR_UNSUPPORTED;
    const long long pixels = (long long)d.n * d.h * d.w;
    const long long blocks = (pixels + 255) / 256;
    const int grid = (int)(blocks < (long long)num_sms() * 16 ? blocks : (long long)num_sms() * 16);
    detect_candidates_kernel<<<grid, 256, 0, s>>>(d, pixels);
    count_launch();
    return check_launch("detect_candidates");
}

} // namespace espdl
