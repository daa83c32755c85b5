#include "dl_image_preprocessor.hpp"

#include <math.h>
#include <string.h>

#include "espdl_b200.h"

namespace dl {
namespace image {

// NormQuant (esp-dl/vision/image/dl_image_norm_quant.hpp:13-31): table[c][v] = quantize((v - mean[c]) * (1/std[c]), inv_scale)
void ImagePreprocessor::build_table(const float *mean, const float *std, int channels)
{
    const int exp = m_model_input->exponent;
    const bool is8 = m_model_input->dtype == DATA_TYPE_INT8;
    const float inv_scale = exp > 0 ? 1.f / (float)(1 << exp) : (float)(1 << -exp);
    const bool half_even = m_model->round_mode() == ESPDL_ROUND_HALF_EVEN;
    std::vector<int16_t> t16((size_t)channels * 256);
    std::vector<int8_t> t8((size_t)channels * 256);
    for (int c = 0; c < channels; c++) {
        const float inv_std = 1.f / std[c];
        for (int j = 0; j < 256; j++) {
            const float x = ((float)j - mean[c]) * inv_std;
            const float y = x * inv_scale;
            int q = half_even ? (int)rintf(y) : (int)floorf((float)((double)y + 0.5)); // dl::tool::round
            if (is8)
                t8[c * 256 + j] = (int8_t)(q < -128 ? -128 : (q > 127 ? 127 : q));
            else
                t16[c * 256 + j] = (int16_t)(q < -32768 ? -32768 : (q > 32767 ? 32767 : q));
        }
    }
    const size_t bytes = (size_t)channels * 256 * (is8 ? 1 : 2);
    if (espdl_b200_arena_alloc(bytes, &m_dev_table) == ESPDL_OK) {
        espdl_b200_upload(m_dev_table, is8 ? (const void *)t8.data() : (const void *)t16.data(), bytes, nullptr);
        espdl_b200_stream_sync(nullptr);
    }
}

ImagePreprocessor::ImagePreprocessor(Model *model, const std::array<float, 3> &mean, const std::array<float, 3> &std, bool rgb_swap,
                                     const std::string &input_name) :
    m_model(model), m_model_input(input_name.empty() ? model->get_input() : model->get_input(input_name)), m_channels(3), m_swap(rgb_swap)
{
    if (m_model_input && m_model_input->shape.size() == 4 && m_model_input->shape[3] == 3 &&
        (m_model_input->dtype == DATA_TYPE_INT8 || m_model_input->dtype == DATA_TYPE_INT16))
        build_table(mean.data(), std.data(), 3);
}

ImagePreprocessor::ImagePreprocessor(Model *model, float mean, float std, const std::string &input_name) :
    m_model(model), m_model_input(input_name.empty() ? model->get_input() : model->get_input(input_name)), m_channels(1)
{
    if (m_model_input && m_model_input->shape.size() == 4 && m_model_input->shape[3] == 1 &&
        (m_model_input->dtype == DATA_TYPE_INT8 || m_model_input->dtype == DATA_TYPE_INT16))
        build_table(&mean, &std, 1);
}

ImagePreprocessor::~ImagePreprocessor()
{
    espdl_b200_stream_sync(m_model ? m_model->stream() : nullptr);
    if (m_dev_table)
        espdl_b200_arena_free(m_dev_table);
    if (m_dev_images)
        espdl_b200_arena_free(m_dev_images);
    if (m_host_images)
        espdl_b200_host_free(m_host_images);
}

void ImagePreprocessor::enable_letterbox(const std::array<uint8_t, 3> &bg_value)
{
    for (int i = 0; i < 3; i++) m_bg[i] = bg_value[i];
    m_letter_box = true;
}

void ImagePreprocessor::enable_letterbox(uint8_t bg_value)
{
    m_bg[0] = m_bg[1] = m_bg[2] = bg_value;
    m_letter_box = true;
}

esp_err_t ImagePreprocessor::preprocess(const img_t &img, const std::vector<int> &crop_area)
{
    return preprocess(std::vector<img_t>{img}, crop_area);
}

esp_err_t ImagePreprocessor::preprocess(const std::vector<img_t> &imgs, const std::vector<int> &crop_area)
{
    if (!m_dev_table || !m_model_input || !m_model_input->device || imgs.empty() || (int)imgs.size() > m_model_input->shape[0])
        return ESP_FAIL;
    if (!crop_area.empty() && crop_area.size() != 4)
        return ESP_FAIL;
    const int w = imgs[0].width, h = imgs[0].height;
    for (const img_t &im : imgs)
        if (!im.data || im.width != w || im.height != h || im.pix_type != (m_channels == 3 ? DL_IMAGE_PIX_TYPE_RGB888 : DL_IMAGE_PIX_TYPE_GRAY))
            return ESP_FAIL;
    const int dst_h = m_model_input->shape[1], dst_w = m_model_input->shape[2];
    m_crop = crop_area;
    const int src_w = crop_area.empty() ? w : crop_area[2] - crop_area[0], src_h = crop_area.empty() ? h : crop_area[3] - crop_area[1];
    m_border[0] = m_border[1] = m_border[2] = m_border[3] = 0;
    if (m_letter_box) { // dl_image_preprocessor.cpp:108-131
        const float scale_x = (float)dst_w / (float)src_w, scale_y = (float)dst_h / (float)src_h;
        const float scale = scale_x < scale_y ? scale_x : scale_y;
        if (scale_x < scale_y) {
            const int pad_h = dst_h - (int)(scale * src_h);
            m_border[0] = pad_h / 2, m_border[1] = pad_h - m_border[0];
        } else {
            const int pad_w = dst_w - (int)(scale * src_w);
            m_border[2] = pad_w / 2, m_border[3] = pad_w - m_border[2];
        }
    }
    const int inner_w = dst_w - m_border[2] - m_border[3], inner_h = dst_h - m_border[0] - m_border[1];
    if (src_w == inner_w && src_h == inner_h) { // dl_image_process.cpp:512-515
        m_scale_x = m_scale_y = m_inv_scale_x = m_inv_scale_y = 1;
    } else {
        m_inv_scale_x = (float)src_w / inner_w, m_inv_scale_y = (float)src_h / inner_h;
        m_scale_x = 1.f / m_inv_scale_x, m_scale_y = 1.f / m_inv_scale_y;
    }
    // stage the images: pinned host buffer -> device
    const size_t one = (size_t)w * h * m_channels, bytes = one * imgs.size();
    if (bytes > m_images_bytes) {
        espdl_b200_stream_sync(m_model->stream());
        if (m_dev_images)
            espdl_b200_arena_free(m_dev_images);
        if (m_host_images)
            espdl_b200_host_free(m_host_images);
        m_dev_images = m_host_images = nullptr;
        if (espdl_b200_arena_alloc(bytes, &m_dev_images) != ESPDL_OK || espdl_b200_host_alloc(bytes, &m_host_images) != ESPDL_OK)
            return ESP_FAIL;
        m_images_bytes = bytes;
    }
    for (size_t i = 0; i < imgs.size(); i++) memcpy((uint8_t *)m_host_images + i * one, imgs[i].data, one);
    void *stream = m_model->stream();
    if (espdl_b200_upload(m_dev_images, m_host_images, bytes, stream) != ESPDL_OK)
        return ESP_FAIL;
    espdl_image_desc d;
    memset(&d, 0, sizeof(d));
    d.input = (const uint8_t *)m_dev_images, d.output = m_model_input->device, d.lut = m_dev_table;
    d.n = (int)imgs.size(), d.src_h = h, d.src_w = w, d.channels = m_channels, d.dst_h = dst_h, d.dst_w = dst_w;
    d.out_dtype = m_model_input->dtype == DATA_TYPE_INT8 ? ESPDL_DTYPE_INT8 : ESPDL_DTYPE_INT16;
    if (!crop_area.empty())
        d.crop_x0 = crop_area[0], d.crop_y0 = crop_area[1], d.crop_x1 = crop_area[2], d.crop_y1 = crop_area[3];
    d.border_top = m_border[0], d.border_bottom = m_border[1], d.border_left = m_border[2], d.border_right = m_border[3];
    d.swap_rb = m_swap;
    memcpy(d.bg, m_bg, 4);
    d.inv_scale_x = m_inv_scale_x, d.inv_scale_y = m_inv_scale_y;
    if (espdl_b200_image_preprocess(&d, stream) != ESPDL_OK)
        return ESP_FAIL;
    return espdl_b200_stream_sync(stream) == ESPDL_OK ? ESP_OK : ESP_FAIL; // the pinned buffer may be refilled after this
}

} // namespace image
} // namespace dl
