#include "dl_model_base.hpp"
#include "dl_module_ops.hpp"
#include "espdl_b200.h"

#include <algorithm>
#include <climits>
#include <cstring>

namespace dl {

// ----------------------------------------------------------------------------- arena planner
size_t MemoryManagerGreedy::plan(std::vector<TensorInfo> &tensors, bool reuse)
{
    constexpr size_t ALIGN = 256;
    auto round_up = [](size_t v) { return (v + ALIGN - 1) / ALIGN * ALIGN; };
    // a buffer lives as long as any tensor that aliases it
    std::vector<int> root(tensors.size());
    for (size_t i = 0; i < tensors.size(); i++) {
        int r = (int)i;
        while (tensors[r].alias_of >= 0) r = tensors[r].alias_of;
        root[i] = r;
    }
    std::vector<int> last(tensors.size()), first(tensors.size());
    std::vector<size_t> bytes(tensors.size());
    for (size_t i = 0; i < tensors.size(); i++) last[i] = tensors[i].last, first[i] = tensors[i].first, bytes[i] = round_up(tensors[i].bytes);
    for (size_t i = 0; i < tensors.size(); i++) {
        last[root[i]] = std::max(last[root[i]], tensors[i].last);
        first[root[i]] = std::min(first[root[i]], tensors[i].first); // a slice may be written before the tensor it lives in
        if (!tensors[i].row_stride) // a slice lies inside its root
            bytes[root[i]] = std::max(bytes[root[i]], round_up(tensors[i].bytes));
    }
    struct Chunk {
        size_t offset, size;
    };
    std::vector<Chunk> free_list;
    size_t arena = 0;
    // roots in order of first use; release buffers whose last reader is before the current step
    std::vector<int> order;
    for (size_t i = 0; i < tensors.size(); i++)
        if (root[i] == (int)i)
            order.push_back((int)i);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return first[a] < first[b]; });
    std::vector<int> live;
    for (int t : order) {
        if (reuse) {
            for (size_t k = 0; k < live.size();) {
                if (last[live[k]] < first[t]) {
                    Chunk c{tensors[live[k]].offset, bytes[live[k]]};
                    // coalesce with neighbours
                    for (size_t f = 0; f < free_list.size();) {
                        if (free_list[f].offset + free_list[f].size == c.offset) {
                            c.offset = free_list[f].offset, c.size += free_list[f].size;
                            free_list.erase(free_list.begin() + f);
                        } else if (c.offset + c.size == free_list[f].offset) {
                            c.size += free_list[f].size;
                            free_list.erase(free_list.begin() + f);
                        } else {
                            f++;
                        }
                    }
                    free_list.push_back(c);
                    live.erase(live.begin() + k);
                } else {
                    k++;
                }
            }
        }
        // best fit
        int best = -1;
        for (size_t f = 0; f < free_list.size(); f++)
            if (free_list[f].size >= bytes[t] && (best < 0 || free_list[f].size < free_list[best].size))
                best = (int)f;
        if (best >= 0) {
            tensors[t].offset = free_list[best].offset;
            if (free_list[best].size == bytes[t]) {
                free_list.erase(free_list.begin() + best);
            } else {
                free_list[best].offset += bytes[t];
                free_list[best].size -= bytes[t];
            }
        } else {
            // grow: extend a free chunk that ends at the arena's end, else append
            int tail = -1;
            for (size_t f = 0; f < free_list.size(); f++)
                if (free_list[f].offset + free_list[f].size == arena)
                    tail = (int)f;
            if (tail >= 0) {
                tensors[t].offset = free_list[tail].offset;
                arena = free_list[tail].offset + bytes[t];
                free_list.erase(free_list.begin() + tail);
            } else {
                tensors[t].offset = arena;
                arena += bytes[t];
            }
        }
        live.push_back(t);
    }
    for (size_t i = 0; i < tensors.size(); i++) {
        if (root[i] == (int)i)
            continue;
        size_t off = tensors[root[i]].offset;
        for (int r = (int)i; tensors[r].alias_of >= 0; r = tensors[r].alias_of) off += tensors[r].view_offset;
        tensors[i].offset = off;
    }
    return arena;
}

// A tensor's device copy into a dense host buffer, also when it is a channel slice of a wider tensor.
static void download_dense(void *host, TensorBase *t, void *stream)
{
    if (!t->row_stride) {
        espdl_b200_download(host, t->device, t->get_bytes(), stream);
        return;
    }
    const size_t es = dtype_sizeof(t->dtype), row = (size_t)t->shape.back() * es;
    espdl_b200_download_rows(host, t->device, row, (size_t)t->row_stride * es, row ? t->get_bytes() / row : 0, stream);
}

// ----------------------------------------------------------------------------- model
static bool env_flag(const char *name, bool def)
{
    const char *v = getenv(name);
    return v ? (*v != '0') : def;
}

Model::Model(const char *path, fbs::model_location_type_t location, int max_internal_size, memory_manager_t mm_type, const uint8_t *key,
             bool param_copy, const std::map<std::string, std::vector<int>> &input_shapes)
{
    m_use_graph = env_flag("ESPDL_B200_GRAPH", true);
    if (load(path, location, 0, key, param_copy) == ESP_OK)
        build(max_internal_size, mm_type, false, input_shapes);
}

Model::Model(const char *path, int model_index, fbs::model_location_type_t location, int max_internal_size, memory_manager_t mm_type,
             const uint8_t *key, bool param_copy, const std::map<std::string, std::vector<int>> &input_shapes)
{
    m_use_graph = env_flag("ESPDL_B200_GRAPH", true);
    if (load(path, location, model_index, key, param_copy) == ESP_OK)
        build(max_internal_size, mm_type, false, input_shapes);
}

Model::Model(fbs::FbsModel *fbs_model, int internal_size, memory_manager_t mm_type, const std::map<std::string, std::vector<int>> &input_shapes)
{
    m_use_graph = env_flag("ESPDL_B200_GRAPH", true);
    if (load(fbs_model) == ESP_OK)
        build(internal_size, mm_type, false, input_shapes);
}

void Model::release_pipeline()
{
    if (m_copy_stream)
        espdl_b200_stream_sync(m_copy_stream);
    for (auto &kv : m_in_stage)
        if (kv.second)
            espdl_b200_arena_free(kv.second);
    m_in_stage.clear();
    for (int s = 0; s < 2; s++) {
        for (auto &kv : m_out_stage[s])
            if (kv.second)
                espdl_b200_host_free(kv.second);
        m_out_stage[s].clear();
        if (m_ev_done[s])
            espdl_b200_event_destroy(m_ev_done[s]);
        m_ev_done[s] = nullptr;
    }
    if (m_ev_uploaded)
        espdl_b200_event_destroy(m_ev_uploaded);
    if (m_ev_consumed)
        espdl_b200_event_destroy(m_ev_consumed);
    m_ev_uploaded = m_ev_consumed = nullptr;
    if (m_copy_stream)
        espdl_b200_stream_destroy(m_copy_stream);
    m_copy_stream = nullptr;
    m_submitted = m_collected = 0;
}

void Model::release()
{
    if (m_model_context && m_model_context->stream)
        espdl_b200_stream_sync(m_model_context->stream);
    release_pipeline();
    if (m_graph)
        espdl_b200_graph_destroy(m_graph);
    if (m_graph_head)
        espdl_b200_graph_destroy(m_graph_head);
    if (m_graph_tail)
        espdl_b200_graph_destroy(m_graph_tail);
    m_graph = m_graph_head = m_graph_tail = nullptr;
    for (auto *m : m_execution_plan) delete m;
    m_execution_plan.clear();
    if (m_model_context) {
        for (auto &kv : m_inputs)
            if (kv.second->data && !kv.second->auto_free) {
                espdl_b200_host_free(kv.second->data);
                kv.second->data = nullptr;
            }
        for (auto &kv : m_outputs)
            if (kv.second->data && !kv.second->auto_free) {
                espdl_b200_host_free(kv.second->data);
                kv.second->data = nullptr;
            }
        if (m_model_context->workspace)
            espdl_b200_arena_free(m_model_context->workspace);
        if (m_model_context->stream)
            espdl_b200_stream_destroy(m_model_context->stream);
        delete m_model_context;
        m_model_context = nullptr;
    }
    if (m_arena)
        espdl_b200_arena_free(m_arena);
    m_arena = nullptr;
    m_inputs.clear();
    m_outputs.clear();
}

Model::~Model()
{
    release();
    if (m_own_fbs_model)
        delete m_fbs_model;
    delete m_fbs_loader;
}

esp_err_t Model::load(const char *path, fbs::model_location_type_t location, int model_index, const uint8_t *key, bool param_copy)
{
    m_fbs_loader = new fbs::FbsLoader(path, location);
    fbs::FbsModel *m = m_fbs_loader->load(model_index, key, param_copy);
    if (!m) {
        ESP_LOGE("dl::Model", "Failed to load model.");
        m_status = ESPDL_ERR_INVALID_ARG;
        return ESP_FAIL;
    }
    m_own_fbs_model = true;
    return load(m);
}

esp_err_t Model::load(fbs::FbsModel *fbs_model)
{
    m_fbs_model = fbs_model;
    if (!fbs_model)
        return ESP_FAIL;
    m_name = fbs_model->get_model_name();
    m_version = fbs_model->get_model_version();
    m_doc_string = fbs_model->get_model_doc_string();
    m_model_context = new ModelContext();
    m_model_context->own_tensors = true;
    // rounding follows the chip the model was exported for (esp-dl/dl/dl_define_private.hpp:44-48)
    std::string target = fbs_model->get_model_metadata_prop("target");
    if (const char *env = getenv("ESPDL_B200_TARGET"))
        if (target.empty())
            target = env;
    m_model_context->round_mode = (target == "esp32p4" || target == "esp32s31") ? ROUND_HALF_EVEN : ROUND_HALF_UP;
    if (const char *env = getenv("ESPDL_B200_ROUND"))
        m_model_context->round_mode = strcmp(env, "half_even") == 0 ? ROUND_HALF_EVEN : ROUND_HALF_UP;

    module::ModuleCreator *creator = module::ModuleCreator::get_instance();
    for (const std::string &node : fbs_model->topological_sort()) {
        const std::string op_type = fbs_model->get_operation_type(node);
        module::Module *mod = creator->create(fbs_model, op_type, node);
        if (!mod) {
            ESP_LOGE("dl::Model", "Do not support operation %s (node %s)", op_type.c_str(), node.c_str());
            m_status = ESPDL_ERR_UNSUPPORTED;
            return ESP_FAIL;
        }
        std::vector<std::string> ins, outs;
        fbs_model->get_operation_inputs_and_outputs(node, ins, outs);
        // initializer inputs become parameter tensors of the context, created once per name
        for (size_t i = 0; i < ins.size(); i++) {
            if (fbs_model->is_parameter(ins[i]) && m_model_context->get_tensor_index(ins[i]) < 0) {
                TensorBase *t = fbs_model->get_operation_parameter(node, (int)i);
                if (t)
                    m_model_context->push_back_tensor(t, ins[i]);
            }
        }
        m_execution_plan.push_back(mod);
        m_module_types.push_back(op_type);
        m_module_inputs.push_back(ins);
        m_module_outputs.push_back(outs);
    }
    return ESP_OK;
}

// Add(x, y) where y is produced by a pointwise int8 Conv, is read by nothing else and has the exponent of x and of the
// sum: the conv adds x to its own result (espdl_conv_desc::residual) and writes the Add's output; the Add leaves the
// plan.  ESP-DL's Add of equal exponents is a saturating sum (esp-dl/dl/base/dl_base_add.cpp:8-44), which is what the
// conv epilogue computes.  ESPDL_B200_FOLD_ADD=0 keeps the Add nodes.
// Block fusion: a depthwise 3x3 conv whose input comes from a pointwise conv (optional) and whose output feeds a
// pointwise conv, optionally followed by a residual Add, becomes ONE FusedBlock module (espdl_b200_fused_block);
// the tensors between the stages then never exist in the arena.  Only tensors with a single reader that are not
// graph outputs may disappear.  By default the depthwise -> pointwise pair (and a residual Add behind it) is fused - the
// tensor between them, as large as the depthwise input, never reaches HBM - and the expand conv stays a launch of its
// own (ESPDL_B200_FUSE_DWPW=0 keeps the pair apart); ESPDL_B200_FUSE_BLOCKS=1 also takes the expand conv into the
// launch, which the measurements so far do not reward.
void Model::fuse_blocks()
{
    const bool whole_blocks = env_flag("ESPDL_B200_FUSE_BLOCKS", false);
    if ((!whole_blocks && !env_flag("ESPDL_B200_FUSE_DWPW", false)) || !m_reuse_memory)
        return;
    ModelContext *ctx = m_model_context;
    std::vector<std::string> graph_outputs = m_fbs_model->get_graph_outputs();
    auto is_graph_output = [&](const std::string &n) { return std::find(graph_outputs.begin(), graph_outputs.end(), n) != graph_outputs.end(); };
    auto readers = [&](const std::string &n) {
        int r = 0;
        for (const auto &ins : m_module_inputs)
            for (const std::string &i : ins)
                if (i == n) r++;
        return r;
    };
    auto producer = [&](const std::string &n) {
        for (size_t k = 0; k < m_module_outputs.size(); k++)
            for (const std::string &o : m_module_outputs[k])
                if (o == n) return (int)k;
        return -1;
    };
    auto is_int8 = [&](const std::string &n) { return m_fbs_model->get_value_info_dtype(n) == DATA_TYPE_INT8; };
    auto private_tensor = [&](const std::string &n) { return readers(n) == 1 && !is_graph_output(n) && !m_fbs_model->is_parameter(n) && is_int8(n); };
    for (size_t s = 0; s < m_execution_plan.size(); s++) {
        if (m_module_types[s] != "Conv" || m_module_outputs[s].size() != 1)
            continue;
        module::Conv *dw = dynamic_cast<module::Conv *>(m_execution_plan[s]);
        TensorBase *dwf = m_module_inputs[s].size() > 1 ? ctx->get_tensor(m_module_inputs[s][1]) : nullptr;
        if (!dw || !dw->is_dw3x3() || !dwf || dwf->shape.size() != 4 || dwf->shape[0] != 3 || dwf->shape[1] != 3)
            continue;
        const std::string y1 = m_module_inputs[s][0], y2 = m_module_outputs[s][0];
        if (!private_tensor(y2) || !is_int8(y1))
            continue;
        int P = -1;
        for (size_t k = s + 1; k < m_execution_plan.size() && P < 0; k++)
            if (!m_module_inputs[k].empty() && m_module_inputs[k][0] == y2)
                P = (int)k;
        module::Conv *proj = P >= 0 && m_module_types[P] == "Conv" ? dynamic_cast<module::Conv *>(m_execution_plan[P]) : nullptr;
        if (!proj || !proj->is_pointwise() || m_module_outputs[P].size() != 1 || m_module_inputs[P].size() < 2 ||
            !module::Conv::filter_is_1x1(ctx->get_tensor(m_module_inputs[P][1])))
            continue;
        int E = producer(y1);
        module::Conv *expand = nullptr;
        if (whole_blocks && E >= 0 && E < (int)s && m_module_types[E] == "Conv" && private_tensor(y1) && m_module_outputs[E].size() == 1) {
            expand = dynamic_cast<module::Conv *>(m_execution_plan[E]);
            if (expand && (!expand->is_pointwise() || m_module_inputs[E].size() < 2 ||
                           !module::Conv::filter_is_1x1(ctx->get_tensor(m_module_inputs[E][1]))))
                expand = nullptr;
        }
        if (!expand)
            E = -1;
        const std::string x = expand ? m_module_inputs[E][0] : y1;
        std::string y3 = m_module_outputs[P][0];
        if (!is_int8(x) || !is_int8(y3))
            continue;
        // a residual Add behind the project conv
        int A = -1;
        std::string res;
        if (private_tensor(y3)) {
            for (size_t k = P + 1; k < m_execution_plan.size() && A < 0; k++)
                if (m_module_types[k] == "Add" && m_module_inputs[k].size() == 2 && m_module_outputs[k].size() == 1 &&
                    (m_module_inputs[k][0] == y3 || m_module_inputs[k][1] == y3))
                    A = (int)k;
            if (A >= 0) {
                res = m_module_inputs[A][0] == y3 ? m_module_inputs[A][1] : m_module_inputs[A][0];
                const std::string out = m_module_outputs[A][0];
                const int e3 = m_fbs_model->get_value_info_exponent(y3);
                if (res == y3 || m_fbs_model->is_parameter(res) || !is_int8(res) || !is_int8(out) || m_fbs_model->get_value_info_exponent(res) != e3 ||
                    m_fbs_model->get_value_info_exponent(out) != e3 || m_fbs_model->get_value_info_shape(res) != m_fbs_model->get_value_info_shape(y3))
                    A = -1;
            }
        }
        // does the kernel take these extents?
        const std::vector<int> xs = m_fbs_model->get_value_info_shape(x), hs = m_fbs_model->get_value_info_shape(y1),
                               os = m_fbs_model->get_value_info_shape(y3);
        if (xs.size() != 4 || hs.size() != 4 || os.size() != 4)
            continue;
        espdl_block_desc probe;
        memset(&probe, 0, sizeof(probe));
        probe.dtype = ESPDL_DTYPE_INT8;
        probe.n = xs[0], probe.in_h = xs[1], probe.in_w = xs[2], probe.in_c = xs[3], probe.hidden_c = hs[3];
        probe.out_h = os[1], probe.out_w = os[2], probe.out_c = os[3];
        probe.stride = dw->stride(), probe.pad_top = dw->pads()[0], probe.pad_left = dw->pads()[2];
        probe.reserved[0] = expand ? 1 : 0;
        if (espdl_b200_fused_block_supported(&probe) != ESPDL_OK)
            continue;
        // build the module; each conv remembers how many inputs it had (data + parameters)
        std::vector<std::string> inputs = {x};
        for (int k : {E, (int)s, P}) {
            if (k < 0)
                continue;
            m_execution_plan[k]->m_inputs_index.assign(m_module_inputs[k].size(), -1);
            for (size_t i = 1; i < m_module_inputs[k].size(); i++) inputs.push_back(m_module_inputs[k][i]);
        }
        if (A >= 0)
            inputs.push_back(res);
        module::FusedBlock *fb = new module::FusedBlock(expand, dw, proj, m_fbs_model->get_value_info_exponent(y1),
                                                        m_fbs_model->get_value_info_exponent(y2), A >= 0, m_execution_plan[P]->name);
        const int last = A >= 0 ? A : P;
        const std::string out_name = m_module_outputs[last][0];
        if (A >= 0)
            delete m_execution_plan[A];
        m_execution_plan[last] = fb;
        m_module_types[last] = "FusedBlock";
        m_module_inputs[last] = inputs;
        m_module_outputs[last] = {out_name};
        std::vector<int> gone;
        for (int k : {E, (int)s, P})
            if (k >= 0 && k != last)
                gone.push_back(k);
        std::sort(gone.rbegin(), gone.rend());
        for (int k : gone) {
            m_execution_plan.erase(m_execution_plan.begin() + k);
            m_module_types.erase(m_module_types.begin() + k);
            m_module_inputs.erase(m_module_inputs.begin() + k);
            m_module_outputs.erase(m_module_outputs.begin() + k);
        }
        s = 0; // indices moved: scan again (fused steps are no Conv any more)
    }
}

// A LUT-type node (LUT, Swish, Sigmoid, Tanh, ... exported with a 256-entry int8 table: esp-dl/dl/module/include/
// dl_module_swish.hpp:84-103, dl_module_lut.hpp:50-76) whose input comes from a dense int8 Conv and is read by nothing
// else: the conv applies the table in its epilogue (espdl_conv_desc::lut, held in shared memory by the tile kernels)
// and writes the LUT node's output; the node and the tensor between the two leave the plan.  Exactly the reference's
// arithmetic: requantise and saturate to the intermediate exponent, then table[(uint8)q ^ 0x80]
// (esp-dl/dl/base/dl_base_lut.cpp:10-15).  Only convs the tensor-core tile kernels take (input channels a multiple of
// 16) are folded; ESPDL_B200_FOLD_LUT=0 keeps the nodes.
void Model::fold_luts()
{
    if (!env_flag("ESPDL_B200_FOLD_LUT", true) || !m_reuse_memory)
        return;
    ModelContext *ctx = m_model_context;
    std::vector<std::string> graph_outputs = m_fbs_model->get_graph_outputs();
    auto is_graph_output = [&](const std::string &n) { return std::find(graph_outputs.begin(), graph_outputs.end(), n) != graph_outputs.end(); };
    for (size_t s = 0; s < m_execution_plan.size(); s++) {
        module::LUT *lut = dynamic_cast<module::LUT *>(m_execution_plan[s]);
        if (!lut || lut->quant_type != QUANT_TYPE_SYMM_8BIT || m_module_inputs[s].empty() || m_module_outputs[s].size() != 1)
            continue;
        TensorBase *table = lut->get_table();
        if (!table || table->dtype != DATA_TYPE_INT8 || table->get_size() != 256)
            continue;
        const std::string x = m_module_inputs[s][0], y = m_module_outputs[s][0];
        if (is_graph_output(x) || m_fbs_model->is_parameter(x) || m_fbs_model->get_value_info_dtype(x) != DATA_TYPE_INT8 ||
            m_fbs_model->get_value_info_dtype(y) != DATA_TYPE_INT8)
            continue;
        int producer = -1, readers = 0;
        for (size_t k = 0; k < m_execution_plan.size(); k++) {
            for (const std::string &o : m_module_outputs[k])
                if (o == x) producer = (int)k;
            for (const std::string &i : m_module_inputs[k])
                if (i == x) readers++;
        }
        if (producer < 0 || producer >= (int)s || readers != 1 || m_module_types[producer] != "Conv" || m_module_outputs[producer].size() != 1 ||
            m_module_inputs[producer].size() < 2)
            continue;
        module::Conv *conv = dynamic_cast<module::Conv *>(m_execution_plan[producer]);
        TensorBase *filter = ctx->get_tensor(m_module_inputs[producer][1]);
        // the kernels that apply a table in their staged epilogue: the tile kernels (Cin a multiple of 16) and the two
        // banded-filter kernels (3x3 with 3 or 8 input channels)
        if (!conv || !conv->can_fuse_lut() || !filter || filter->shape.size() != 4)
            continue;
        const bool banded = filter->shape[0] == 3 && filter->shape[1] == 3 && (filter->shape[2] == 3 || filter->shape[2] == 8);
        if (filter->shape[2] % 16 != 0 && !banded)
            continue;
        conv->set_fused_lut(lut->release_table(), m_fbs_model->get_value_info_exponent(x));
        m_module_outputs[producer][0] = y;
        delete m_execution_plan[s];
        m_execution_plan.erase(m_execution_plan.begin() + s);
        m_module_types.erase(m_module_types.begin() + s);
        m_module_inputs.erase(m_module_inputs.begin() + s);
        m_module_outputs.erase(m_module_outputs.begin() + s);
        s--;
    }
}

void Model::fold_prelus()
{
    if (!env_flag("ESPDL_B200_FOLD_PRELU", true) || !m_reuse_memory)
        return;
    ModelContext *ctx = m_model_context;
    std::vector<std::string> graph_outputs = m_fbs_model->get_graph_outputs();
    auto is_graph_output = [&](const std::string &n) { return std::find(graph_outputs.begin(), graph_outputs.end(), n) != graph_outputs.end(); };
    for (size_t s = 0; s < m_execution_plan.size(); s++) {
        module::PRelu *act = dynamic_cast<module::PRelu *>(m_execution_plan[s]);
        if (!act || act->quant_type != QUANT_TYPE_SYMM_8BIT || m_module_inputs[s].empty() || m_module_outputs[s].size() != 1)
            continue;
        TensorBase *alpha = act->get_table();
        const std::string x = m_module_inputs[s][0], y = m_module_outputs[s][0];
        if (!alpha || alpha->dtype != DATA_TYPE_INT8 || !alpha->data || is_graph_output(x) || m_fbs_model->is_parameter(x) ||
            m_fbs_model->get_value_info_dtype(x) != DATA_TYPE_INT8 || m_fbs_model->get_value_info_dtype(y) != DATA_TYPE_INT8)
            continue;
        int producer = -1, readers = 0;
        for (size_t k = 0; k < m_execution_plan.size(); k++) {
            for (const std::string &o : m_module_outputs[k])
                if (o == x) producer = (int)k;
            for (const std::string &i : m_module_inputs[k])
                if (i == x) readers++;
        }
        if (producer < 0 || producer >= (int)s || readers != 1 || m_module_types[producer] != "Conv" || m_module_outputs[producer].size() != 1 ||
            m_module_inputs[producer].size() < 2)
            continue;
        module::Conv *conv = dynamic_cast<module::Conv *>(m_execution_plan[producer]);
        TensorBase *filter = ctx->get_tensor(m_module_inputs[producer][1]);
        if (!conv || !conv->can_fuse_channel_tables() || !filter || filter->shape.size() != 4)
            continue;
        const int channels = conv->is_depthwise() ? filter->shape[2] * filter->shape[3] : filter->shape[3];
        if (alpha->get_size() != channels)
            continue;
        // dl::base::prelu (esp-dl/dl/base/dl_base_prelu.cpp:7-21): a value below zero becomes (value * slope) >> shift with a
        // plain arithmetic shift, shift = e_out - e_in - e_slope (a left shift when negative); the rest passes unchanged
        const int shift = m_fbs_model->get_value_info_exponent(y) - m_fbs_model->get_value_info_exponent(x) - (int)alpha->exponent;
        if (shift > 30 || shift < -16)
            continue;
        std::vector<int8_t> tables((size_t)channels * 256);
        const int8_t *slope = (const int8_t *)alpha->data;
        for (int c = 0; c < channels; c++)
            for (int i = 0; i < 256; i++) {
                const int q = (int)(int8_t)(uint8_t)(i ^ 0x80);
                int v = q;
                if (q < 0) {
                    const int prod = q * (int)slope[c];
                    v = shift > 0 ? (prod >> shift) : (int)((unsigned)prod << (-shift));
                    v = std::max(-128, std::min(127, v));
                }
                tables[(size_t)c * 256 + i] = (int8_t)v;
            }
        TensorBase *t = new TensorBase({channels * 256}, tables.data(), 0, DATA_TYPE_INT8, true);
        conv->set_fused_channel_tables(t, m_fbs_model->get_value_info_exponent(x));
        m_module_outputs[producer][0] = y;
        delete m_execution_plan[s];
        m_execution_plan.erase(m_execution_plan.begin() + s);
        m_module_types.erase(m_module_types.begin() + s);
        m_module_inputs.erase(m_module_inputs.begin() + s);
        m_module_outputs.erase(m_module_outputs.begin() + s);
        s--;
    }
}

void Model::fold_quantize_after_softmax()
{
    if (!env_flag("ESPDL_B200_FOLD_QUANT", true) || !m_reuse_memory)
        return;
    std::vector<std::string> graph_outputs = m_fbs_model->get_graph_outputs();
    auto is_graph_output = [&](const std::string &n) { return std::find(graph_outputs.begin(), graph_outputs.end(), n) != graph_outputs.end(); };
    for (size_t s = 0; s < m_execution_plan.size(); s++) {
        if (m_module_types[s] != "QuantizeLinear" || m_module_inputs[s].empty() || m_module_outputs[s].size() != 1)
            continue;
        const std::string x = m_module_inputs[s][0], y = m_module_outputs[s][0];
        const dtype_t yt = m_fbs_model->get_value_info_dtype(y);
        if (is_graph_output(x) || m_fbs_model->get_value_info_dtype(x) != DATA_TYPE_FLOAT || (yt != DATA_TYPE_INT8 && yt != DATA_TYPE_INT16))
            continue;
        int producer = -1, readers = 0;
        for (size_t k = 0; k < m_execution_plan.size(); k++) {
            for (const std::string &o : m_module_outputs[k])
                if (o == x) producer = (int)k;
            for (const std::string &i : m_module_inputs[k])
                if (i == x) readers++;
        }
        if (producer < 0 || producer >= (int)s || readers != 1 || m_module_outputs[producer].size() != 1 ||
            (m_module_types[producer] != "Softmax" && m_module_types[producer] != "LogSoftmax"))
            continue;
        m_module_outputs[producer][0] = y;
        delete m_execution_plan[s];
        m_execution_plan.erase(m_execution_plan.begin() + s);
        m_module_types.erase(m_module_types.begin() + s);
        m_module_inputs.erase(m_module_inputs.begin() + s);
        m_module_outputs.erase(m_module_outputs.begin() + s);
        s--;
    }
}

void Model::fold_residual_adds()
{
    if (!env_flag("ESPDL_B200_FOLD_ADD", true) || !m_reuse_memory)
        return; // with every tensor kept (tests that read intermediates) the graph stays as exported
    std::vector<std::string> graph_outputs = m_fbs_model->get_graph_outputs();
    auto is_graph_output = [&](const std::string &n) { return std::find(graph_outputs.begin(), graph_outputs.end(), n) != graph_outputs.end(); };
    for (size_t s = 0; s < m_execution_plan.size(); s++) {
        if (m_module_types[s] != "Add" || m_module_inputs[s].size() != 2 || m_module_outputs[s].size() != 1)
            continue;
        const std::string out = m_module_outputs[s][0];
        for (int which = 0; which < 2; which++) {
            const std::string y = m_module_inputs[s][which], x = m_module_inputs[s][1 - which];
            if (x == y || m_fbs_model->is_parameter(x) || m_fbs_model->is_parameter(y) || is_graph_output(y))
                continue;
            int producer = -1, x_producer = -1, readers = 0;
            for (size_t k = 0; k < m_execution_plan.size(); k++) {
                for (const std::string &o : m_module_outputs[k]) {
                    if (o == y) producer = (int)k;
                    if (o == x) x_producer = (int)k;
                }
                for (const std::string &i : m_module_inputs[k])
                    if (i == y) readers++;
            }
            if (producer < 0 || producer >= (int)s || readers != 1 || m_module_types[producer] != "Conv" || x_producer >= producer)
                continue;
            module::Conv *conv = dynamic_cast<module::Conv *>(m_execution_plan[producer]);
            if (!conv || !conv->can_fold_add() || m_module_outputs[producer].size() != 1 || m_module_inputs[producer].size() < 2 ||
                !module::Conv::filter_is_1x1(m_model_context->get_tensor(m_module_inputs[producer][1])))
                continue; // only a [1,1,Cin,Cout] filter: the kernels that add a residual are the pointwise ones
            if (m_fbs_model->get_value_info_dtype(x) != DATA_TYPE_INT8 || m_fbs_model->get_value_info_dtype(y) != DATA_TYPE_INT8 ||
                m_fbs_model->get_value_info_dtype(out) != DATA_TYPE_INT8)
                continue;
            const int ex = m_fbs_model->get_value_info_exponent(x), ey = m_fbs_model->get_value_info_exponent(y);
            if (ex != ey || ex != m_fbs_model->get_value_info_exponent(out))
                continue;
            if (m_fbs_model->get_value_info_shape(x) != m_fbs_model->get_value_info_shape(y))
                continue;
            conv->set_residual();
            m_module_inputs[producer].push_back(x);
            m_module_outputs[producer][0] = out;
            delete m_execution_plan[s];
            m_execution_plan.erase(m_execution_plan.begin() + s);
            m_module_types.erase(m_module_types.begin() + s);
            m_module_inputs.erase(m_module_inputs.begin() + s);
            m_module_outputs.erase(m_module_outputs.begin() + s);
            s--;
            break;
        }
    }
}

// Concat and Split along the last axis without the copy: an input of a Concat whose producer can write rows a stride
// apart is placed inside the Concat's output (the producer writes its channels of every row directly), and an output
// of a Split whose consumers can read such rows is a window into the Split's input.  Both need every other consumer of
// the slice to read strided rows too; offsets, widths and strides are whole 16-byte units.  A tensor is a slice of one
// wider tensor at most, and a tensor that holds slices is not itself a slice.  Returns how many tensors became slices.
int Model::alias_channel_slices(std::vector<TensorInfo> &infos, std::map<std::string, int> &info_index,
                                const std::vector<std::vector<std::vector<int>>> &step_in_shapes, std::vector<bool> &is_root)
{
    // Slices start, end and stride on 32-byte boundaries: a 16-byte slice of a 48-byte row would be read and written as half
    // sectors, which costs its elementwise producers more than the copy it saves (measured on the detector's first C3k2 block).
    constexpr long long SLICE_UNIT = 32;
    const int steps = (int)m_execution_plan.size();
    std::vector<std::vector<std::pair<int, int>>> consumers(infos.size()); // (step, input position)
    for (int step = 0; step < steps; step++)
        for (size_t i = 0; i < m_module_inputs[step].size(); i++) {
            auto it = info_index.find(m_module_inputs[step][i]);
            if (it != info_index.end())
                consumers[it->second].push_back({step, (int)i});
        }
    std::vector<bool> is_view(infos.size(), false);
    auto readers_ok = [&](int t, int but_step) {
        for (const auto &c : consumers[t])
            if (c.first != but_step && !m_execution_plan[c.first]->strided_input_ok(c.second, step_in_shapes[c.first]))
                return false;
        return true;
    };
    int made = 0;
    for (int step = 0; step < steps; step++) {
        module::Module *mod = m_execution_plan[step];
        if (module::Concat *cat = dynamic_cast<module::Concat *>(mod)) {
            auto oit = info_index.find(m_module_outputs[step][0]);
            if (oit == info_index.end())
                continue;
            const int out = oit->second;
            const int nd = (int)infos[out].shape.size();
            const int ax = cat->get_axis() < 0 ? cat->get_axis() + nd : cat->get_axis();
            const long long es = (long long)dtype_sizeof(infos[out].dtype);
            if (nd < 2 || ax != nd - 1 || is_view[out] || infos[out].alias_of >= 0 || (infos[out].shape[ax] * es) % SLICE_UNIT != 0)
                continue;
            long long off = 0;
            for (size_t i = 0; i < m_module_inputs[step].size(); i++) {
                const std::string &in_name = m_module_inputs[step][i];
                const long long ci = step_in_shapes[step][i].empty() ? 0 : step_in_shapes[step][i].back();
                auto it = info_index.find(in_name);
                const long long at = off;
                off += ci;
                if (it == info_index.end())
                    continue;
                const int t = it->second;
                TensorInfo &ti = infos[t];
                if (ti.is_graph_io || ti.first < 0 || is_view[t] || is_root[t] || ti.alias_of >= 0 || ti.dtype != infos[out].dtype ||
                    (at * es) % SLICE_UNIT != 0 || (ci * es) % SLICE_UNIT != 0 || (int)ti.shape.size() != nd)
                    continue;
                if (std::count(m_module_inputs[step].begin(), m_module_inputs[step].end(), in_name) != 1)
                    continue;
                const std::vector<std::string> &pouts = m_module_outputs[ti.first];
                const int o_pos = (int)(std::find(pouts.begin(), pouts.end(), in_name) - pouts.begin());
                if (!m_execution_plan[ti.first]->strided_output_ok(o_pos, step_in_shapes[ti.first]) || !readers_ok(t, step))
                    continue;
                ti.alias_of = out, ti.view_offset = (size_t)(at * es), ti.row_stride = infos[out].shape[ax];
                is_view[t] = true, is_root[out] = true;
                made++;
            }
        } else if (module::Split *sp = dynamic_cast<module::Split *>(mod)) {
            auto xit = info_index.find(m_module_inputs[step][0]);
            if (xit == info_index.end())
                continue;
            const int x = xit->second;
            const int nd = (int)infos[x].shape.size();
            const int ax = sp->get_axis() < 0 ? sp->get_axis() + nd : sp->get_axis();
            const long long es = (long long)dtype_sizeof(infos[x].dtype);
            if (nd < 2 || ax != nd - 1 || is_view[x] || infos[x].alias_of >= 0 || (infos[x].shape[ax] * es) % SLICE_UNIT != 0)
                continue;
            long long off = 0;
            for (size_t o = 0; o < m_module_outputs[step].size(); o++) {
                auto it = info_index.find(m_module_outputs[step][o]);
                if (it == info_index.end())
                    break;
                const int t = it->second;
                TensorInfo &ti = infos[t];
                const long long co = ti.shape.empty() ? 0 : ti.shape.back();
                const long long at = off;
                off += co;
                if (ti.is_graph_io || ti.last == INT_MAX || is_view[t] || is_root[t] || ti.alias_of >= 0 || (at * es) % SLICE_UNIT != 0 || (co * es) % SLICE_UNIT != 0 ||
                    consumers[t].empty() || !mod->strided_output_ok((int)o, step_in_shapes[step]) || !readers_ok(t, -1))
                    continue;
                ti.alias_of = x, ti.view_offset = (size_t)(at * es), ti.row_stride = infos[x].shape[ax];
                is_view[t] = true, is_root[x] = true;
                made++;
            }
        }
    }
    return made;
}

void Model::build(size_t max_internal_size, memory_manager_t mm_type, bool preload, const std::map<std::string, std::vector<int>> &input_shapes)
{
    (void)max_internal_size;
    (void)mm_type;
    (void)preload;
    if (!m_fbs_model || !m_model_context || m_built)
        return;
    fuse_blocks();
    fold_luts();
    fold_prelus();
    fold_quantize_after_softmax();
    fold_residual_adds();
    ModelContext *ctx = m_model_context;
    std::vector<TensorInfo> &infos = m_tensor_infos;
    std::map<std::string, int> info_index;
    auto add_info = [&](const std::string &name, const std::vector<int> &shape, int first) {
        TensorInfo ti;
        ti.name = name, ti.shape = shape, ti.first = first, ti.last = first;
        ti.dtype = m_fbs_model->get_value_info_dtype(name);
        if (ti.dtype == DATA_TYPE_UNDEFINED)
            ti.dtype = DATA_TYPE_INT8;
        ti.exponent = m_fbs_model->get_value_info_exponent(name);
        size_t n = 1;
        for (int d : shape) n *= (size_t)d;
        ti.bytes = n * dtype_sizeof(ti.dtype);
        infos.push_back(ti);
        info_index[name] = (int)infos.size() - 1;
        return (int)infos.size() - 1;
    };
    for (const std::string &name : m_fbs_model->get_graph_inputs()) {
        std::vector<int> shape = m_fbs_model->get_value_info_shape(name);
        auto it = input_shapes.find(name);
        if (it != input_shapes.end())
            shape = it->second;
        // Graph inputs keep their buffer for the model's lifetime (the reference lets later tensors reuse it):
        // the plan can then be replayed on device-resident inputs without another upload.
        TensorInfo &ti = infos[add_info(name, shape, -1)];
        ti.is_graph_io = true;
        ti.last = INT_MAX;
    }
    // shape inference, lifetimes and in-place links along the plan
    std::vector<std::vector<std::vector<int>>> step_in_shapes;
    for (size_t step = 0; step < m_execution_plan.size(); step++) {
        module::Module *mod = m_execution_plan[step];
        std::vector<std::vector<int>> in_shapes;
        for (const std::string &in : m_module_inputs[step]) {
            auto it = info_index.find(in);
            if (it != info_index.end()) {
                in_shapes.push_back(infos[it->second].shape);
                infos[it->second].last = std::max(infos[it->second].last, (int)step);
            } else if (TensorBase *p = ctx->get_tensor(in)) {
                in_shapes.push_back(p->shape);
            } else {
                in_shapes.push_back({});
            }
        }
        bool shapes_known = true;
        for (size_t i = 0; i < in_shapes.size(); i++) {
            if (in_shapes[i].empty() && !m_module_inputs[step][i].empty() && !ctx->get_tensor(m_module_inputs[step][i])) {
                ESP_LOGE("Model", "%s %s: input %s has no producer, no value_info shape and is no parameter", m_module_types[step].c_str(),
                         mod->name ? mod->name : "?", m_module_inputs[step][i].c_str());
                shapes_known = false;
            }
        }
        if (!shapes_known) {
            m_status = ESPDL_ERR_INVALID_ARG;
            return;
        }
        std::vector<std::vector<int>> out_shapes = mod->get_output_shape(in_shapes);
        for (size_t o = 0; o < m_module_outputs[step].size() && o < out_shapes.size(); o++)
            add_info(m_module_outputs[step][o], out_shapes[o], (int)step);
        step_in_shapes.push_back(in_shapes);
    }
    for (const std::string &name : m_fbs_model->get_graph_outputs()) {
        auto it = info_index.find(name);
        if (it != info_index.end()) {
            infos[it->second].last = INT_MAX;
            infos[it->second].is_graph_io = true;
        }
    }
    // In-place: a view (Reshape / Flatten / ...) always shares its input's buffer; a module that may overwrite an
    // input (Add, LUT, RequantizeLinear, ...) takes the buffer of an input that dies at this step, is no graph
    // input/output, is not shared through a view, and is large enough (dl_memory_manager_greedy.cpp:147-212).
    std::vector<bool> slice_root(infos.size(), false);
    if (env_flag("ESPDL_B200_SLICE_VIEWS", true))
        m_slice_views = alias_channel_slices(infos, info_index, step_in_shapes, slice_root);
    if (m_reuse_memory) {
        std::vector<bool> has_view = slice_root; // nothing is overwritten in a buffer that holds slices
        for (size_t step = 0; step < m_execution_plan.size(); step++) {
            module::Module *mod = m_execution_plan[step];
            if (mod->inplace == MODULE_NON_INPLACE || m_module_outputs[step].size() != 1)
                continue;
            const int out = info_index[m_module_outputs[step][0]];
            if (infos[out].row_stride)
                continue; // the output is a slice of a Concat output: it has its place already
            for (const std::string &in_name : m_module_inputs[step]) {
                auto it = info_index.find(in_name);
                if (it == info_index.end())
                    continue;
                TensorInfo &in = infos[it->second];
                if (mod->inplace == MODULE_INPLACE_UNCHANGED_BUFFER) {
                    if (!in.is_graph_io || infos[out].last != INT_MAX) {
                        infos[out].alias_of = it->second;
                        has_view[it->second] = true;
                        int r = it->second;
                        while (infos[r].alias_of >= 0) r = infos[r].alias_of;
                        has_view[r] = true;
                    }
                    break;
                }
                int r = it->second;
                while (infos[r].alias_of >= 0) r = infos[r].alias_of;
                bool root_dies = true; // every tensor on this buffer must be dead after this step
                for (size_t k = 0; k < infos.size(); k++) {
                    int rk = (int)k;
                    while (infos[rk].alias_of >= 0) rk = infos[rk].alias_of;
                    if (rk == r && (int)k != out && infos[k].last > (int)step)
                        root_dies = false;
                }
                // equal element sizes only: the kernels run one thread per element, and an output element of another
                // width would land on input elements that other threads have not read yet (float Softmax -> int8)
                if (root_dies && !in.is_graph_io && !infos[r].is_graph_io && !has_view[r] && infos[out].last != INT_MAX &&
                    in.bytes >= infos[out].bytes && in.dtype == infos[out].dtype) {
                    infos[out].alias_of = it->second;
                    break;
                }
            }
        }
    }
    m_arena_bytes = MemoryManagerGreedy::plan(infos, m_reuse_memory);
    // the last step that reads a graph input's buffer (directly, or through a view / slice that lives in it)
    m_input_steps = 0;
    for (size_t i = 0; i < infos.size(); i++) {
        int r = (int)i;
        while (infos[r].alias_of >= 0) r = infos[r].alias_of;
        if (infos[r].first >= 0)
            continue;
        for (size_t step = 0; step < m_execution_plan.size(); step++)
            for (const std::string &in : m_module_inputs[step])
                if (in == infos[i].name)
                    m_input_steps = std::max(m_input_steps, (int)step + 1);
    }
    if (m_plan_only)
        return;
    if (espdl_b200_arena_alloc(m_arena_bytes + 256, &m_arena) != ESPDL_OK) {
        ESP_LOGE("dl::Model", "Failed to allocate a %.1f MB device arena", m_arena_bytes / 1048576.0);
        m_status = ESPDL_ERR_NO_MEM;
        return;
    }
    espdl_b200_memset(m_arena, 0, m_arena_bytes, nullptr);
    espdl_b200_stream_create(&ctx->stream);
    for (TensorInfo &ti : infos) {
        TensorBase *t = new TensorBase(ti.shape, nullptr, ti.exponent, ti.dtype, false);
        t->device = (char *)m_arena + ti.offset;
        t->row_stride = ti.row_stride;
        if (ti.is_graph_io) { // pinned host buffer the user reads / writes
            void *h = nullptr;
            if (espdl_b200_host_alloc(t->get_aligned_bytes(), &h) == ESPDL_OK) {
                memset(h, 0, t->get_aligned_bytes());
                t->data = h;
            }
        }
        ctx->push_back_tensor(t, ti.name);
        if (ti.first < 0)
            m_inputs[ti.name] = t;
        else if (ti.last == INT_MAX)
            m_outputs[ti.name] = t;
    }
    size_t ws = 0;
    for (size_t step = 0; step < m_execution_plan.size(); step++) {
        module::Module *mod = m_execution_plan[step];
        mod->m_inputs_index.clear();
        mod->m_outputs_index.clear();
        for (const std::string &in : m_module_inputs[step]) mod->m_inputs_index.push_back(ctx->get_tensor_index(in));
        for (const std::string &out : m_module_outputs[step]) mod->m_outputs_index.push_back(ctx->get_tensor_index(out));
        if (mod->prepare(ctx) != ESP_OK) {
            ESP_LOGE("dl::Model", "prepare failed for node %s", mod->name ? mod->name : "?");
            m_status = ESPDL_ERR_CUDA;
            return;
        }
        ws = std::max(ws, mod->workspace_bytes(ctx));
    }
    if (ws) {
        if (espdl_b200_arena_alloc(ws, &ctx->workspace) != ESPDL_OK) {
            m_status = ESPDL_ERR_NO_MEM;
            return;
        }
        ctx->workspace_bytes = ws;
    }
    espdl_b200_stream_sync(nullptr);
    m_built = true;
}

esp_err_t Model::execute(int first, int last)
{
    ModelContext *ctx = m_model_context;
    for (int i = first; i < last; i++) {
        m_execution_plan[i]->forward(ctx, RUNTIME_MODE_SINGLE_CORE);
        if (ctx->status) {
            m_status = ctx->status;
            return ESP_FAIL;
        }
    }
    return ESP_OK;
}

esp_err_t Model::run_device(bool sync)
{
    if (!m_built)
        return ESP_FAIL;
    ModelContext *ctx = m_model_context;
    int st = ESPDL_OK;
    if (m_use_graph) {
        if (!m_graph) {
            // one plain pass first (it also settles lazily created state), then capture the same launches
            if (execute(0, (int)m_execution_plan.size()) != ESP_OK || espdl_b200_stream_sync(ctx->stream) != ESPDL_OK)
                return ESP_FAIL;
            st = espdl_b200_graph_begin(ctx->stream);
            if (!st) {
                esp_err_t e = execute(0, (int)m_execution_plan.size());
                st = espdl_b200_graph_end(ctx->stream, &m_graph);
                if (e != ESP_OK)
                    st = m_status;
            }
            if (st) {
                m_status = st;
                return ESP_FAIL;
            }
        }
        st = espdl_b200_graph_launch(m_graph, ctx->stream);
    } else if (execute(0, (int)m_execution_plan.size()) != ESP_OK) {
        return ESP_FAIL;
    }
    if (!st && sync)
        st = espdl_b200_stream_sync(ctx->stream);
    if (st)
        m_status = st;
    return st ? ESP_FAIL : ESP_OK;
}

// One of the two parts of a pipelined pass on the model's stream: steps [0, m_input_steps) or the rest, replayed as a
// captured graph of its own when graphs are in use.
esp_err_t Model::run_part(bool head)
{
    ModelContext *ctx = m_model_context;
    const int first = head ? 0 : m_input_steps, last = head ? m_input_steps : (int)m_execution_plan.size();
    if (first >= last)
        return ESP_OK;
    if (!m_use_graph)
        return execute(first, last);
    void *&graph = head ? m_graph_head : m_graph_tail;
    int st = ESPDL_OK;
    if (!graph) {
        st = espdl_b200_graph_begin(ctx->stream);
        if (!st) {
            esp_err_t e = execute(first, last);
            st = espdl_b200_graph_end(ctx->stream, &graph);
            if (e != ESP_OK)
                st = m_status ? m_status : ESPDL_ERR_CUDA;
        }
    }
    if (!st)
        st = espdl_b200_graph_launch(graph, ctx->stream);
    if (st)
        m_status = st;
    return st ? ESP_FAIL : ESP_OK;
}

void Model::run(runtime_mode_t mode)
{
    (void)mode;
    if (!m_built)
        return;
    ModelContext *ctx = m_model_context;
    for (auto &kv : m_inputs)
        if (kv.second->data)
            espdl_b200_upload(kv.second->device, kv.second->data, kv.second->get_bytes(), ctx->stream);
    if (run_device(false) != ESP_OK)
        return;
    for (auto &kv : m_outputs)
        if (kv.second->data)
            espdl_b200_download(kv.second->data, kv.second->device, kv.second->get_bytes(), ctx->stream);
    int st = espdl_b200_stream_sync(ctx->stream);
    if (st)
        m_status = st;
}

esp_err_t Model::submit()
{
    if (!m_built || m_submitted - m_collected >= 2)
        return ESP_FAIL;
    ModelContext *ctx = m_model_context;
    int st = ESPDL_OK;
    // Upload straight into the input tensors when the plan has steps that never read them (see m_input_steps)
    const bool direct = m_input_steps > 0 && m_input_steps < (int)m_execution_plan.size() && env_flag("ESPDL_B200_DIRECT_UPLOAD", true);
    if (!m_copy_stream) {
        // first use: second stream, events, a device staging buffer per input (unless uploads go direct), two pinned slots per output
        st = espdl_b200_stream_create(&m_copy_stream);
        if (!st) st = espdl_b200_event_create(&m_ev_uploaded);
        if (!st) st = espdl_b200_event_create(&m_ev_consumed);
        for (int s = 0; s < 2 && !st; s++) st = espdl_b200_event_create(&m_ev_done[s]);
        for (auto &kv : m_inputs)
            if (!st && !direct)
                st = espdl_b200_arena_alloc(kv.second->get_bytes(), &m_in_stage[kv.first]);
        for (int s = 0; s < 2; s++)
            for (auto &kv : m_outputs)
                if (!st)
                    st = espdl_b200_host_alloc(kv.second->get_bytes(), &m_out_stage[s][kv.first]);
        if (!st && !m_graph && m_use_graph) // capture the plan before the first pipelined pass
            st = run_device(true) == ESP_OK ? ESPDL_OK : (m_status ? m_status : ESPDL_ERR_CUDA);
    }
    // upload on the copy stream as soon as the previous submission no longer needs the destination: its staging buffers
    // copied out, or (direct) its steps that read the input tensors finished
    if (!st && m_submitted > 0)
        st = espdl_b200_stream_wait_event(m_copy_stream, m_ev_consumed);
    for (auto &kv : m_inputs)
        if (!st && kv.second->data)
            st = espdl_b200_upload(direct ? kv.second->device : m_in_stage[kv.first], kv.second->data, kv.second->get_bytes(), m_copy_stream);
    if (!st) st = espdl_b200_event_record(m_ev_uploaded, m_copy_stream);
    if (!st) st = espdl_b200_event_sync(m_ev_uploaded); // the host buffers are free again when submit() returns
    // plan on the compute stream: (staging -> input tensors,) forward pass, outputs -> this submission's pinned slot
    if (!st) st = espdl_b200_stream_wait_event(ctx->stream, m_ev_uploaded);
    if (direct) {
        if (!st && run_part(true) != ESP_OK)
            st = m_status ? m_status : ESPDL_ERR_CUDA;
        if (!st) st = espdl_b200_event_record(m_ev_consumed, ctx->stream);
        if (!st && run_part(false) != ESP_OK)
            st = m_status ? m_status : ESPDL_ERR_CUDA;
    } else {
        for (auto &kv : m_inputs)
            if (!st)
                st = espdl_b200_device_copy(kv.second->device, m_in_stage[kv.first], kv.second->get_bytes(), ctx->stream);
        if (!st) st = espdl_b200_event_record(m_ev_consumed, ctx->stream);
        if (!st && run_device(false) != ESP_OK)
            st = m_status ? m_status : ESPDL_ERR_CUDA;
    }
    const int slot = (int)(m_submitted & 1);
    for (auto &kv : m_outputs)
        if (!st)
            st = espdl_b200_download(m_out_stage[slot][kv.first], kv.second->device, kv.second->get_bytes(), ctx->stream);
    if (!st) st = espdl_b200_event_record(m_ev_done[slot], ctx->stream);
    if (st) {
        m_status = st;
        return ESP_FAIL;
    }
    m_submitted++;
    return ESP_OK;
}

esp_err_t Model::wait()
{
    if (m_collected >= m_submitted)
        return ESP_FAIL;
    const int slot = (int)(m_collected & 1);
    int st = espdl_b200_event_sync(m_ev_done[slot]);
    if (!st)
        for (auto &kv : m_outputs)
            if (kv.second->data)
                memcpy(kv.second->data, m_out_stage[slot][kv.first], kv.second->get_bytes());
    m_collected++;
    if (!st && m_collected == m_submitted) // queue drained: a good moment to pick up a kernel's bounded-wait status
        st = espdl_b200_stream_sync(m_model_context->stream);
    if (st) {
        m_status = st;
        return ESP_FAIL;
    }
    return ESP_OK;
}

void Model::run(TensorBase *input, runtime_mode_t mode)
{
    if (m_inputs.size() != 1 || !input)
        return;
    m_inputs.begin()->second->assign(input); // copy / quantise into the graph input, as the reference does
    run(mode);
}

void Model::run(std::map<std::string, TensorBase *> &user_inputs, runtime_mode_t mode, std::map<std::string, TensorBase *> user_outputs)
{
    for (auto &kv : user_inputs) {
        TensorBase *t = get_input(kv.first);
        if (t)
            t->assign(kv.second);
    }
    run(mode);
    for (auto &kv : user_outputs) {
        TensorBase *t = get_intermediate(kv.first);
        if (t && kv.second && kv.second->data && t->device) {
            if (t->row_stride && kv.second->get_bytes() >= t->get_bytes())
                download_dense(kv.second->data, t, m_model_context->stream);
            else if (!t->row_stride)
                espdl_b200_download(kv.second->data, t->device, std::min(kv.second->get_bytes(), t->get_bytes()), m_model_context->stream);
            espdl_b200_stream_sync(m_model_context->stream);
        }
    }
}

void Model::run(int stage_num, int stage_index, runtime_mode_t mode)
{
    (void)mode;
    if (!m_built || stage_num <= 0 || stage_index < 0 || stage_index >= stage_num)
        return;
    ModelContext *ctx = m_model_context;
    const int n = (int)m_execution_plan.size();
    const int per = (n + stage_num - 1) / stage_num;
    const int first = stage_index * per, last = std::min(n, first + per);
    if (stage_index == 0)
        for (auto &kv : m_inputs)
            if (kv.second->data)
                espdl_b200_upload(kv.second->device, kv.second->data, kv.second->get_bytes(), ctx->stream);
    execute(first, last);
    if (stage_index == stage_num - 1)
        for (auto &kv : m_outputs)
            if (kv.second->data)
                espdl_b200_download(kv.second->data, kv.second->device, kv.second->get_bytes(), ctx->stream);
    espdl_b200_stream_sync(ctx->stream);
}

// The model's own golden check (esp-dl/dl/model/src/dl_model_base.cpp:442-519): feed the embedded test inputs,
// run module by module, compare every output that has an embedded expected value.
esp_err_t Model::test()
{
    if (!m_built)
        return ESP_FAIL;
    ModelContext *ctx = m_model_context;
    for (auto &kv : m_inputs) {
        TensorBase *t = m_fbs_model->get_test_input_tensor(kv.first);
        if (!t) {
            ESP_LOGE("dl::Model", "Model input %s doesn't have a corresponding test input.", kv.first.c_str());
            return ESP_FAIL;
        }
        const bool ok = t->get_bytes() == kv.second->get_bytes();
        if (ok) {
            memcpy(kv.second->data, t->data, t->get_bytes());
            espdl_b200_upload(kv.second->device, kv.second->data, kv.second->get_bytes(), ctx->stream);
        }
        delete t;
        if (!ok) {
            ESP_LOGE("dl::Model", "test input %s does not match the (batch-overridden?) input shape", kv.first.c_str());
            return ESP_FAIL;
        }
    }
    esp_err_t result = ESP_OK;
    for (size_t step = 0; step < m_execution_plan.size(); step++) {
        if (execute((int)step, (int)step + 1) != ESP_OK)
            return ESP_FAIL;
        for (const std::string &out_name : m_module_outputs[step]) {
            TensorBase *expect = m_fbs_model->get_test_output_tensor(out_name);
            if (!expect)
                continue;
            TensorBase *got_dev = ctx->get_tensor(out_name);
            TensorBase got(got_dev->shape, nullptr, (int)got_dev->exponent, got_dev->dtype, true);
            download_dense(got.data, got_dev, ctx->stream);
            espdl_b200_stream_sync(ctx->stream);
            if (!got.equal(expect, 2e-5f, true)) {
                ESP_LOGE("dl::Model", "Test failed for output %s of %s", out_name.c_str(), m_module_types[step].c_str());
                result = ESP_FAIL;
            }
            delete expect;
        }
    }
    if (espdl_b200_stream_sync(ctx->stream) != ESPDL_OK)
        return ESP_FAIL;
    return result;
}

std::map<std::string, module_info> Model::get_module_info()
{
    std::map<std::string, module_info> info;
    if (!m_built)
        return info;
    ModelContext *ctx = m_model_context;
    void *e0 = nullptr, *e1 = nullptr;
    espdl_b200_event_create(&e0);
    espdl_b200_event_create(&e1);
    execute(0, (int)m_execution_plan.size()); // warm up
    espdl_b200_stream_sync(ctx->stream);
    for (size_t step = 0; step < m_execution_plan.size(); step++) {
        float best = 1e30f;
        for (int rep = 0; rep < 3; rep++) {
            espdl_b200_event_record(e0, ctx->stream);
            execute((int)step, (int)step + 1);
            espdl_b200_event_record(e1, ctx->stream);
            float ms = 0;
            espdl_b200_event_elapsed_ms(e0, e1, &ms);
            best = std::min(best, ms);
        }
        char key[32];
        snprintf(key, sizeof(key), "%04d:", (int)step);
        module_info mi;
        mi.type = m_module_types[step];
        mi.latency_us = best * 1000.f;
        info[std::string(key) + (m_execution_plan[step]->name ? m_execution_plan[step]->name : "")] = mi;
    }
    espdl_b200_event_destroy(e0);
    espdl_b200_event_destroy(e1);
    return info;
}

void Model::profile_module(bool sort_module_by_latency)
{
    auto info = get_module_info();
    std::vector<std::pair<std::string, module_info>> rows(info.begin(), info.end());
    if (sort_module_by_latency)
        std::sort(rows.begin(), rows.end(), [](auto &a, auto &b) { return a.second.latency_us > b.second.latency_us; });
    float total = 0;
    printf("%-72s %-20s %12s\n", "name", "type", "latency(us)");
    for (auto &r : rows) {
        printf("%-72s %-20s %12.1f\n", r.first.c_str(), r.second.type.c_str(), r.second.latency_us);
        total += r.second.latency_us;
    }
    printf("%-72s %-20s %12.1f\n", "total", "", total);
}

void Model::profile_memory()
{
    size_t params = 0;
    for (auto *t : m_model_context->m_variables)
        if (t && t->device_owned)
            params += t->get_aligned_bytes();
    printf("device arena (activations): %.2f MB\nparameters on device: %.2f MB\nflatbuffers model: %.2f MB\nscratch: %.2f MB\n",
           m_arena_bytes / 1048576.0, params / 1048576.0, m_fbs_model ? m_fbs_model->get_size() / 1048576.0 : 0.0,
           m_model_context->workspace_bytes / 1048576.0);
}

void Model::minimize()
{
    if (!m_model_context)
        return;
    for (TensorBase *t : m_model_context->m_variables) {
        // parameters that live on the device: the kernels read that copy; operands of a few bytes (Clip bounds, Resize
        // scales, Mul scalars) are read on the host at every forward and stay
        if (t && t->device && t->device_owned && t->data && t->auto_free && t->get_aligned_bytes() > 256) {
            free(t->data);
            t->data = nullptr;
        }
    }
    if (m_fbs_model)
        m_fbs_model->clear_map();
    module::ModuleCreator::get_instance()->clear();
}

void Model::profile(bool sort_module_by_latency)
{
    profile_memory();
    profile_module(sort_module_by_latency);
}

TensorBase *Model::get_input(const std::string &name)
{
    auto it = m_inputs.find(name);
    return it == m_inputs.end() ? nullptr : it->second;
}

TensorBase *Model::get_output(const std::string &name)
{
    auto it = m_outputs.find(name);
    return it == m_outputs.end() ? nullptr : it->second;
}

TensorBase *Model::get_intermediate(const std::string &name) { return m_model_context ? m_model_context->get_tensor(name) : nullptr; }

std::string Model::get_metadata_prop(const std::string &key) { return m_fbs_model ? m_fbs_model->get_model_metadata_prop(key) : ""; }

void Model::print()
{
    for (size_t i = 0; i < m_execution_plan.size(); i++) {
        fprintf(stderr, "%3d %-18s %s\n", (int)i, m_module_types[i].c_str(), m_execution_plan[i]->name ? m_execution_plan[i]->name : "");
        m_execution_plan[i]->print();
    }
}

void Model::reset()
{
    for (auto *m : m_execution_plan) m->reset();
}

} // namespace dl
