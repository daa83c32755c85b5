// dl::cls::ClsPostprocessor of the reference (esp-dl/vision/classification/dl_cls_postprocessor.cpp:6-52): softmax over
// the model's int8 logits (the Softmax module, here its device kernel), score threshold, sort by score, top-k.  The
// logits stay in HBM until the float scores come back; sorting a thousand floats per image stays on the host, as in
// the reference.  Addition: results are per image of the batch, and carry the category index next to the name.
#pragma once
#include <string>
#include <vector>

#include "dl_model_base.hpp"
#include "dl_module_ops.hpp"

namespace dl {
namespace cls {

typedef struct {
    const char *cat_name; ///< from the table given with set_category_names(), else null
    float score;
    int category;
} result_t;

class ClsPostprocessor {
public:
    ClsPostprocessor(Model *model, const int top_k, const float score_thr, bool need_softmax, const std::string &output_name = "");
    virtual ~ClsPostprocessor();
    void set_topk(int topk) { m_topk = topk; }
    void set_score_thr(float score_thr) { m_score_thr = score_thr; }
    void set_category_names(const char *const *names) { m_cat_names = names; }
    /// Image 0 of the batch (the reference's call).
    std::vector<result_t> &postprocess() { return postprocess(0); }
    /// Any image of the batch; the scores of the whole batch are computed and fetched once per model run
    /// (call invalidate() after each run).
    std::vector<result_t> &postprocess(int image);
    void invalidate() { m_valid = false; }

protected:
    Model *m_model;
    TensorBase *m_model_output;
    TensorBase *m_output = nullptr; ///< float scores, device buffer + host copy
    module::Softmax *m_softmax_module = nullptr;
    int m_topk;
    float m_score_thr;
    bool m_need_softmax, m_valid = false;
    const char *const *m_cat_names = nullptr;
    std::vector<result_t> m_cls_result;
};

} // namespace cls
} // namespace dl
