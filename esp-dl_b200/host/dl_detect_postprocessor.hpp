// dl::detect::yolo11PostProcessor of the reference (esp-dl/vision/detect/dl_detect_yolo11_postprocessor.cpp,
// dl_detect_postprocessor.cpp): candidates above the score threshold from three heads, boxes decoded from the 4 x 16
// distribution codes (DFL integral), sigmoid scores, sorted, NMS, top-k.  The scan over H x W x classes runs on the
// device (espdl_b200_detect_candidates); the candidates (a few hundred records) are decoded, sorted and suppressed here
// with the reference's float arithmetic, so results are the reference's bit for bit.  Addition: one result list per
// image of the batch.
#pragma once
#include <list>
#include <string>
#include <vector>

#include "dl_image_preprocessor.hpp"
#include "dl_model_base.hpp"

namespace dl {
namespace detect {

struct result_t {
    int category;
    float score;
    std::vector<int> box;      ///< [left_up_x, left_up_y, right_down_x, right_down_y]
    std::vector<int> keypoint; ///< unused by this post-processor
    void limit_box(int width, int height);
};

typedef struct {
    int stride_y, stride_x, offset_y, offset_x;
} anchor_point_stage_t;

class yolo11PostProcessor {
public:
    yolo11PostProcessor(Model *model, dl::image::ImagePreprocessor *image_preprocessor, const float score_thr, const float nms_thr,
                        const int top_k, const std::vector<anchor_point_stage_t> &stages);
    ~yolo11PostProcessor();
    /// Names of the (box, score) outputs per stage; the reference looks up "box0"/"score0" ... "box2"/"score2".
    void set_output_names(const std::vector<std::pair<std::string, std::string>> &names) { m_names = names; }
    void set_score_thr(float v) { m_score_thr = v; }
    void set_nms_thr(float v) { m_nms_thr = v; }
    void clear_result();
    esp_err_t postprocess();
    std::list<result_t> &get_result(int width, int height, int image = 0);

private:
    void nms(std::list<result_t> &boxes);
    Model *m_model;
    dl::image::ImagePreprocessor *m_image_preprocessor;
    float m_score_thr, m_nms_thr;
    int m_top_k;
    std::vector<anchor_point_stage_t> m_stages;
    std::vector<std::pair<std::string, std::string>> m_names;
    std::vector<std::list<result_t>> m_box_lists; ///< per image
    void *m_dev_records = nullptr, *m_dev_count = nullptr;
    int m_capacity = 0;
};

} // namespace detect
} // namespace dl
