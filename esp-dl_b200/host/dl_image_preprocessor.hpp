// dl::image::ImagePreprocessor of the reference (esp-dl/vision/image/dl_image_preprocessor.hpp:9-47) on the B200
// backend: same constructor arguments, letterbox switch, getters and preprocess() call; the image bytes are host
// memory (as on the ESP32), the conversion runs on the device (espdl_b200_image_preprocess) and writes straight into
// the model's input tensor in HBM.  Additions: a batch of equally sized images fills the batch slots of the input in
// one launch.  Only what the forward path needs is kept: RGB888 and GRAY sources, nearest-neighbour resize (the
// reference's default path); the warp-affine overload and the RGB565 / HSV pixel types are not built.
#pragma once
#include <array>
#include <string>
#include <vector>

#include "dl_model_base.hpp"

namespace dl {
namespace image {

typedef enum { DL_IMAGE_PIX_TYPE_RGB888 = 0, DL_IMAGE_PIX_TYPE_GRAY = 1 } pix_type_t;

typedef struct {
    void *data; ///< host pointer, height x width x channels bytes
    uint16_t width;
    uint16_t height;
    pix_type_t pix_type;
} img_t;

class ImagePreprocessor {
public:
    ImagePreprocessor(Model *model, const std::array<float, 3> &mean, const std::array<float, 3> &std, bool rgb_swap = false,
                      const std::string &input_name = "");
    ImagePreprocessor(Model *model, float mean, float std, const std::string &input_name = "");
    ~ImagePreprocessor();
    void enable_letterbox(const std::array<uint8_t, 3> &bg_value = {});
    void enable_letterbox(uint8_t bg_value = 0);
    float get_resize_scale_x(bool inv = false) { return inv ? m_inv_scale_x : m_scale_x; }
    float get_resize_scale_y(bool inv = false) { return inv ? m_inv_scale_y : m_scale_y; }
    int get_crop_area_top_left_x() { return m_crop.empty() ? 0 : m_crop[0]; }
    int get_crop_area_top_left_y() { return m_crop.empty() ? 0 : m_crop[1]; }
    int get_border_top() { return m_border[0]; }
    int get_border_left() { return m_border[2]; }
    TensorBase *get_model_input() { return m_model_input; }
    /// One image into batch slot 0 (the reference's call).  Returns ESP_OK / ESP_FAIL instead of aborting.
    esp_err_t preprocess(const img_t &img, const std::vector<int> &crop_area = {});
    /// One image per batch slot, all of one size and pixel type; imgs.size() must not exceed the input's batch.
    esp_err_t preprocess(const std::vector<img_t> &imgs, const std::vector<int> &crop_area = {});

private:
    void build_table(const float *mean, const float *std, int channels);
    Model *m_model;
    TensorBase *m_model_input;
    int m_channels;
    bool m_swap = false, m_letter_box = false;
    uint8_t m_bg[4] = {0, 0, 0, 0};
    std::vector<int> m_crop;
    int m_border[4] = {0, 0, 0, 0};
    float m_scale_x = 0, m_scale_y = 0, m_inv_scale_x = 0, m_inv_scale_y = 0;
    void *m_dev_table = nullptr, *m_dev_images = nullptr, *m_host_images = nullptr;
    size_t m_images_bytes = 0;
};

} // namespace image
} // namespace dl
