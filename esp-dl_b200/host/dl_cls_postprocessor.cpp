#include "dl_cls_postprocessor.hpp"

#include <algorithm>

#include "espdl_b200.h"

namespace dl {
namespace cls {

ClsPostprocessor::ClsPostprocessor(Model *model, const int top_k, const float score_thr, bool need_softmax, const std::string &output_name) :
    m_model(model), m_model_output(output_name.empty() ? model->get_output() : model->get_output(output_name)), m_topk(top_k),
    m_score_thr(score_thr), m_need_softmax(need_softmax)
{
    if (!m_model_output)
        return;
    m_output = new TensorBase(m_model_output->shape, nullptr, 0, DATA_TYPE_FLOAT);
    if (espdl_b200_arena_alloc(m_output->get_aligned_bytes(), &m_output->device) == ESPDL_OK)
        m_output->device_owned = true;
    if (need_softmax)
        m_softmax_module = new module::Softmax(nullptr, -1, MODULE_NON_INPLACE, QUANT_TYPE_SYMM_8BIT);
}

ClsPostprocessor::~ClsPostprocessor()
{
    delete m_softmax_module;
    delete m_output;
}

std::vector<result_t> &ClsPostprocessor::postprocess(int image)
{
    m_cls_result.clear();
    if (!m_model_output || !m_output || !m_output->device || !m_output->data || m_model_output->shape.empty())
        return m_cls_result;
    const int batch = m_model_output->shape[0];
    const int classes = m_model_output->get_size() / (batch > 0 ? batch : 1);
    if (image < 0 || image >= batch)
        return m_cls_result;
    if (!m_valid) {
        espdl_b200_stream_sync(m_model->stream());
        if (m_need_softmax) {
            m_softmax_module->run(m_model_output, m_output); // device kernel, float scores
        } else {
            // TensorBase::assign of an int8 tensor to a float one: q * 2^exponent (dl_tensor_base.cpp:223-404)
            std::vector<int8_t> q((size_t)m_model_output->get_size());
            espdl_b200_download(q.data(), m_model_output->device, q.size(), nullptr);
            espdl_b200_stream_sync(nullptr);
            const int e = m_model_output->exponent;
            const float scale = e > 0 ? (float)(1 << e) : 1.f / (float)(1 << -e);
            for (size_t i = 0; i < q.size(); i++) ((float *)m_output->data)[i] = (float)q[i] * scale;
        }
        if (m_need_softmax) {
            espdl_b200_download(m_output->data, m_output->device, m_output->get_bytes(), nullptr);
            espdl_b200_stream_sync(nullptr);
        }
        m_valid = true;
    }
    const float *scores = (const float *)m_output->data + (size_t)image * classes;
    for (int i = 0; i < classes; i++)
        if (scores[i] > m_score_thr)
            m_cls_result.push_back({m_cat_names ? m_cat_names[i] : nullptr, scores[i], i});
    std::sort(m_cls_result.begin(), m_cls_result.end(), [](const result_t &a, const result_t &b) { return a.score > b.score; });
    if ((int)m_cls_result.size() > m_topk)
        m_cls_result.resize(m_topk);
    return m_cls_result;
}

} // namespace cls
} // namespace dl
