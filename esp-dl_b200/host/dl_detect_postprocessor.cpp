#include "dl_detect_postprocessor.hpp"

#include <algorithm>
#include <math.h>
#include <string.h>

#include "espdl_b200.h"

namespace dl {
namespace detect {

namespace {
// dl::math (esp-dl/dl/math/include/dl_math.hpp:200-258), same expressions and evaluation types
inline float sigmoid(float x) { return 1.0 / (1.0 + expf(-x)); }
inline float inverse_sigmoid(float x) { return -logf(1.0 / x - 1); }
inline void softmax(float *x, int num)
{
    float max_input = x[0];
    for (int i = 1; i < num; i++) max_input = max_input > x[i] ? max_input : x[i];
    float sum = 0;
    for (int i = 0; i < num; i++) {
        x[i] = expf(x[i] - max_input);
        sum += x[i];
    }
    for (int i = 0; i < num; i++) x[i] /= sum;
}
inline float dfl_integral(float *data, int reg_max)
{
    softmax(data, reg_max + 1);
    float sum = 0;
    for (int i = 0; i <= reg_max; i++) sum += data[i] * i;
    return sum;
}
inline float scale_of(int e) { return e > 0 ? (float)(1 << e) : 1.f / (float)(1 << -e); }
} // namespace

void result_t::limit_box(int width, int height)
{
    box[0] = std::min(std::max(box[0], 0), width - 1);
    box[1] = std::min(std::max(box[1], 0), height - 1);
    box[2] = std::min(std::max(box[2], 0), width - 1);
    box[3] = std::min(std::max(box[3], 0), height - 1);
}

yolo11PostProcessor::yolo11PostProcessor(Model *model, dl::image::ImagePreprocessor *image_preprocessor, const float score_thr,
                                         const float nms_thr, const int top_k, const std::vector<anchor_point_stage_t> &stages) :
    m_model(model), m_image_preprocessor(image_preprocessor), m_score_thr(score_thr), m_nms_thr(nms_thr), m_top_k(top_k), m_stages(stages)
{
    for (size_t i = 0; i < stages.size(); i++) m_names.push_back({"box" + std::to_string(i), "score" + std::to_string(i)});
}

yolo11PostProcessor::~yolo11PostProcessor()
{
    if (m_dev_records)
        espdl_b200_arena_free(m_dev_records);
    if (m_dev_count)
        espdl_b200_arena_free(m_dev_count);
}

void yolo11PostProcessor::clear_result() { m_box_lists.clear(); }

esp_err_t yolo11PostProcessor::postprocess()
{
    clear_result();
    void *stream = m_model->stream();
    std::vector<TensorBase *> boxes, scores;
    for (size_t i = 0; i < m_stages.size(); i++) {
        boxes.push_back(m_model->get_output(m_names[i].first));
        scores.push_back(m_model->get_output(m_names[i].second));
        if (!boxes[i] || !scores[i] || !boxes[i]->device || !scores[i]->device || scores[i]->dtype != DATA_TYPE_INT8 ||
            boxes[i]->dtype != DATA_TYPE_INT8 || scores[i]->shape.size() != 4 || boxes[i]->shape.size() != 4 || boxes[i]->shape[3] != 64)
            return ESP_FAIL;
    }
    const int batch = scores[0]->shape[0];
    m_box_lists.resize(batch);
    if (!m_dev_count && espdl_b200_arena_alloc(16, &m_dev_count) != ESPDL_OK)
        return ESP_FAIL;
    std::vector<espdl_detect_record> records;
    for (int attempt = 0; attempt < 2; attempt++) {
        if (!m_dev_records) {
            if (m_capacity == 0)
                m_capacity = 4096 * batch;
            if (espdl_b200_arena_alloc((size_t)m_capacity * sizeof(espdl_detect_record), &m_dev_records) != ESPDL_OK)
                return ESP_FAIL;
        }
        espdl_b200_memset(m_dev_count, 0, 16, stream);
        for (size_t i = 0; i < m_stages.size(); i++) {
            espdl_detect_desc d;
            memset(&d, 0, sizeof(d));
            d.score = (const int8_t *)scores[i]->device, d.box = (const int8_t *)boxes[i]->device;
            d.records = (espdl_detect_record *)m_dev_records, d.count = (uint32_t *)m_dev_count;
            d.n = batch, d.h = scores[i]->shape[1], d.w = scores[i]->shape[2], d.classes = scores[i]->shape[3], d.box_channels = 64;
            // T score_thr_quant = quantize<T>(inverse_sigmoid(score_thr), 1 / score_exp)  (dl_detect_yolo11_postprocessor.cpp:24)
            const float inv = 1.f / scale_of(scores[i]->exponent);
            int q = (int)floorf((float)((double)(inverse_sigmoid(m_score_thr) * inv) + 0.5));
            if (m_model->round_mode() == ESPDL_ROUND_HALF_EVEN)
                q = (int)rintf(inverse_sigmoid(m_score_thr) * inv);
            d.score_threshold = std::min(std::max(q, -128), 127);
            d.capacity = m_capacity, d.stage = (int)i;
            if (espdl_b200_detect_candidates(&d, stream) != ESPDL_OK)
                return ESP_FAIL;
        }
        uint32_t count = 0;
        if (espdl_b200_download(&count, m_dev_count, 4, stream) != ESPDL_OK || espdl_b200_stream_sync(stream) != ESPDL_OK)
            return ESP_FAIL;
        if ((int)count > m_capacity) { // more candidates than room: grow once and scan again
            espdl_b200_arena_free(m_dev_records);
            m_dev_records = nullptr;
            m_capacity = (int)count + 1024;
            continue;
        }
        records.resize(count);
        if (count && (espdl_b200_download(records.data(), m_dev_records, (size_t)count * sizeof(espdl_detect_record), stream) != ESPDL_OK ||
                      espdl_b200_stream_sync(stream) != ESPDL_OK))
            return ESP_FAIL;
        break;
    }
    // the reference meets the candidates stage by stage in (y, x, class) order and inserts each behind the boxes of equal
    // or higher score: scan order first, then a stable sort by score
    std::sort(records.begin(), records.end(), [](const espdl_detect_record &a, const espdl_detect_record &b) {
        if (a.image != b.image) return a.image < b.image;
        if (a.stage != b.stage) return a.stage < b.stage;
        if (a.y != b.y) return a.y < b.y;
        if (a.x != b.x) return a.x < b.x;
        return a.category < b.category;
    });
    const float inv_resize_scale_x = m_image_preprocessor ? m_image_preprocessor->get_resize_scale_x(true) : 1.f;
    const float inv_resize_scale_y = m_image_preprocessor ? m_image_preprocessor->get_resize_scale_y(true) : 1.f;
    const int border_left = m_image_preprocessor ? m_image_preprocessor->get_border_left() : 0;
    const int border_top = m_image_preprocessor ? m_image_preprocessor->get_border_top() : 0;
    const int reg_max = 16;
    std::vector<std::vector<result_t>> per_image(batch);
    for (const espdl_detect_record &r : records) {
        const anchor_point_stage_t &st = m_stages[r.stage];
        const float score_exp = scale_of(scores[r.stage]->exponent), box_exp = scale_of(boxes[r.stage]->exponent);
        const int center_y = r.y * st.stride_y + st.offset_y, center_x = r.x * st.stride_x + st.offset_x;
        float box_data[64];
        for (int i = 0; i < reg_max * 4; i++) box_data[i] = (float)r.box[i] * box_exp;
        result_t nb;
        nb.category = r.category;
        nb.score = sigmoid((float)r.score * score_exp);
        nb.box = {(int)(((center_x - dfl_integral(box_data, reg_max - 1) * st.stride_x) - border_left) * inv_resize_scale_x),
                  (int)(((center_y - dfl_integral(box_data + reg_max, reg_max - 1) * st.stride_y) - border_top) * inv_resize_scale_y),
                  (int)(((center_x + dfl_integral(box_data + 2 * reg_max, reg_max - 1) * st.stride_x) - border_left) * inv_resize_scale_x),
                  (int)(((center_y + dfl_integral(box_data + 3 * reg_max, reg_max - 1) * st.stride_y) - border_top) * inv_resize_scale_y)};
        per_image[r.image].push_back(nb);
    }
    for (int b = 0; b < batch; b++) {
        std::stable_sort(per_image[b].begin(), per_image[b].end(), [](const result_t &x, const result_t &y) { return x.score > y.score; });
        m_box_lists[b].assign(per_image[b].begin(), per_image[b].end());
        nms(m_box_lists[b]);
    }
    return ESP_OK;
}

// esp-dl/vision/detect/dl_detect_postprocessor.cpp:5-41
void yolo11PostProcessor::nms(std::list<result_t> &boxes)
{
    int kept_number = 0;
    for (auto kept = boxes.begin(); kept != boxes.end(); kept++) {
        kept_number++;
        if (kept_number >= m_top_k) {
            boxes.erase(++kept, boxes.end());
            break;
        }
        const int kept_area = (kept->box[2] - kept->box[0] + 1) * (kept->box[3] - kept->box[1] + 1);
        auto other = kept;
        other++;
        for (; other != boxes.end();) {
            const int inter_lt_x = std::max(kept->box[0], other->box[0]), inter_lt_y = std::max(kept->box[1], other->box[1]);
            const int inter_rb_x = std::min(kept->box[2], other->box[2]), inter_rb_y = std::min(kept->box[3], other->box[3]);
            const int inter_height = inter_rb_y - inter_lt_y + 1, inter_width = inter_rb_x - inter_lt_x + 1;
            if (inter_height > 0 && inter_width > 0) {
                const int other_area = (other->box[2] - other->box[0] + 1) * (other->box[3] - other->box[1] + 1);
                const int inter_area = inter_height * inter_width;
                const float iou = (float)inter_area / (kept_area + other_area - inter_area);
                if (iou > m_nms_thr) {
                    other = boxes.erase(other);
                    continue;
                }
            }
            other++;
        }
    }
}

std::list<result_t> &yolo11PostProcessor::get_result(int width, int height, int image)
{
    static std::list<result_t> empty;
    if (image < 0 || image >= (int)m_box_lists.size())
        return empty;
    for (result_t &res : m_box_lists[image]) res.limit_box(width, height);
    return m_box_lists[image];
}

} // namespace detect
} // namespace dl
