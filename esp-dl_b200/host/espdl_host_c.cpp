// Flat C wrappers around dl::Model so that Python (tests, bench.py) can drive the C++ host layer through ctypes.
// C++ users include dl_model_base.hpp directly; nothing here adds behaviour.
#include "dl_cls_postprocessor.hpp"
#include "dl_detect_postprocessor.hpp"
#include "dl_image_preprocessor.hpp"
#include "dl_model_base.hpp"
#include "espdl_b200.h"

#include <cstring>
#include <string>

using namespace dl;

namespace {
struct Handle {
    Model *model = nullptr;
    std::vector<std::string> input_names, output_names;
    std::string text;
};

TensorBase *io_tensor(Handle *h, int is_output, int index)
{
    auto &names = is_output ? h->output_names : h->input_names;
    if (index < 0 || index >= (int)names.size())
        return nullptr;
    return is_output ? h->model->get_output(names[index]) : h->model->get_input(names[index]);
}
} // namespace

extern "C" {

/// batch > 0 overrides dim 0 of every graph input.  flags: bit0 = no CUDA graph, bit1 = no buffer reuse.
void *espdl_model_create(const char *path, int batch, int flags)
{
    Handle *h = new Handle();
    Model *m = new Model();
    h->model = m;
    m->m_use_graph = !(flags & 1) && (getenv("ESPDL_B200_GRAPH") ? getenv("ESPDL_B200_GRAPH")[0] != '0' : true);
    m->m_reuse_memory = !(flags & 2);
    if (m->load(path, fbs::MODEL_LOCATION_IN_SDCARD, 0, nullptr, true) != ESP_OK) {
        delete m;
        delete h;
        return nullptr;
    }
    std::map<std::string, std::vector<int>> shapes;
    if (batch > 0) {
        for (const std::string &name : m->get_fbs_model()->get_graph_inputs()) {
            std::vector<int> s = m->get_fbs_model()->get_value_info_shape(name);
            if (!s.empty())
                s[0] = batch;
            shapes[name] = s;
        }
    }
    m->build(0, MEMORY_MANAGER_GREEDY, false, shapes);
    if (m->m_status) {
        delete m;
        delete h;
        return nullptr;
    }
    for (auto &kv : m->get_inputs()) h->input_names.push_back(kv.first);
    for (auto &kv : m->get_outputs()) h->output_names.push_back(kv.first);
    return h;
}

/// Loads a model and plans its arena without touching a device.  Returns the number of planned tensors (negative on
/// error); *arena_bytes and *slices receive the arena size and the number of channel slices, and `text` (capacity `cap`)
/// one line per slice: "name<TAB>name of the tensor it lives in<TAB>byte offset inside it<TAB>row stride in elements".
int espdl_model_plan(const char *path, int batch, int reuse, size_t *arena_bytes, int *slices, char *text, size_t cap)
{
    Model m;
    m.m_plan_only = true;
    m.m_reuse_memory = reuse != 0;
    if (m.load(path, fbs::MODEL_LOCATION_IN_SDCARD, 0, nullptr, true) != ESP_OK)
        return -1;
    std::map<std::string, std::vector<int>> shapes;
    if (batch > 0) {
        for (const std::string &name : m.get_fbs_model()->get_graph_inputs()) {
            std::vector<int> s = m.get_fbs_model()->get_value_info_shape(name);
            if (!s.empty())
                s[0] = batch;
            shapes[name] = s;
        }
    }
    m.build(0, MEMORY_MANAGER_GREEDY, false, shapes);
    if (m.m_status)
        return -2;
    const std::vector<TensorInfo> &infos = m.tensor_infos();
    std::string lines;
    int n_slices = 0;
    for (const TensorInfo &ti : infos)
        if (ti.row_stride) {
            n_slices++;
            lines += ti.name + "\t" + infos[ti.alias_of].name + "\t" + std::to_string(ti.view_offset) + "\t" + std::to_string(ti.row_stride) + "\n";
        }
    if (arena_bytes)
        *arena_bytes = m.arena_bytes();
    if (slices)
        *slices = n_slices;
    if (text && cap) {
        const size_t n = std::min(cap - 1, lines.size());
        memcpy(text, lines.data(), n);
        text[n] = 0;
    }
    return (int)infos.size();
}

void espdl_model_destroy(void *handle)
{
    Handle *h = (Handle *)handle;
    if (h) {
        delete h->model;
        delete h;
    }
}

int espdl_model_num_io(void *handle, int is_output)
{
    Handle *h = (Handle *)handle;
    return (int)(is_output ? h->output_names.size() : h->input_names.size());
}

/// Describes graph input / output `index`: name, shape (up to 8 dims), dtype, exponent, host and device address.
int espdl_model_io_info(void *handle, int is_output, int index, const char **name, int *ndim, int *shape, int *dtype, int *exponent,
                        void **host, void **device)
{
    Handle *h = (Handle *)handle;
    TensorBase *t = io_tensor(h, is_output, index);
    if (!t)
        return ESPDL_ERR_INVALID_ARG;
    *name = (is_output ? h->output_names : h->input_names)[index].c_str();
    *ndim = (int)t->shape.size();
    for (int i = 0; i < *ndim && i < 8; i++) shape[i] = t->shape[i];
    *dtype = (int)t->dtype, *exponent = (int)t->exponent, *host = t->data, *device = t->device;
    return ESPDL_OK;
}

int espdl_model_run(void *handle)
{
    Handle *h = (Handle *)handle;
    h->model->run();
    return h->model->m_status;
}

int espdl_model_run_device(void *handle, int sync)
{
    Handle *h = (Handle *)handle;
    h->model->run_device(sync != 0);
    return h->model->m_status;
}

int espdl_model_submit(void *handle)
{
    Handle *h = (Handle *)handle;
    return h->model->submit() == ESP_OK ? 0 : (h->model->m_status ? h->model->m_status : -1);
}

int espdl_model_wait(void *handle)
{
    Handle *h = (Handle *)handle;
    return h->model->wait() == ESP_OK ? 0 : (h->model->m_status ? h->model->m_status : -1);
}

/// Operator types with a registered creator (dl::module::ModuleCreator), one per line; needs no GPU.
const char *espdl_registered_ops(void)
{
    static std::string text;
    text.clear();
    for (const std::string &op : dl::module::ModuleCreator::get_instance()->registered_ops()) text += op + "\n";
    return text.c_str();
}

/// dl::Model::reset(): clears the state modules keep between runs (the StreamingCache frames).
void espdl_model_reset(void *handle) { ((Handle *)handle)->model->reset(); }

/// dl::Model::minimize(): frees the host copies of device-resident parameters, the name maps and the module registry.
void espdl_model_minimize(void *handle) { ((Handle *)handle)->model->minimize(); }

int espdl_model_test(void *handle) { return ((Handle *)handle)->model->test(); }

void *espdl_model_stream(void *handle) { return ((Handle *)handle)->model->stream(); }

size_t espdl_model_arena_bytes(void *handle) { return ((Handle *)handle)->model->arena_bytes(); }

int espdl_model_num_modules(void *handle) { return (int)((Handle *)handle)->model->num_modules(); }
/// Tensors the planner placed as channel slices inside a Concat output / Split input (no copy).
int espdl_model_num_slice_views(void *handle) { return ((Handle *)handle)->model->num_slice_views(); }

/// Copies the named tensor (any graph tensor; meaningful for intermediates only when built without buffer reuse)
/// to `dst`.  Returns the tensor's byte size, or a negative status.
long long espdl_model_read_tensor(void *handle, const char *name, void *dst, size_t dst_bytes)
{
    Handle *h = (Handle *)handle;
    TensorBase *t = h->model->get_intermediate(name);
    if (!t || !t->device)
        return ESPDL_ERR_INVALID_ARG;
    if (dst) {
        if (dst_bytes < t->get_bytes())
            return ESPDL_ERR_INVALID_ARG;
        int st;
        if (t->row_stride) { // a channel slice of a wider tensor: gather its rows
            const size_t es = dtype_sizeof(t->dtype), row = (size_t)t->shape.back() * es;
            st = espdl_b200_download_rows(dst, t->device, row, (size_t)t->row_stride * es, row ? t->get_bytes() / row : 0, h->model->stream());
        } else {
            st = espdl_b200_download(dst, t->device, t->get_bytes(), h->model->stream());
        }
        if (!st)
            st = espdl_b200_stream_sync(h->model->stream());
        if (st)
            return st;
    }
    return (long long)t->get_bytes();
}

/// dl::detect::yolo11PostProcessor over the outputs named names[2*i] (box) / names[2*i+1] (score) of `stages` heads with
/// strides[i] (offset = stride / 2): results of image `image`, at most `max_results`, as rows {category, x0, y0, x1, y1}
/// in `boxes` and scores in `scores`.  Returns the number of results, -1 on error.
int espdl_model_detect(void *handle, int image, int stages, const char *const *names, const int *strides, float score_thr, float nms_thr,
                       int top_k, int width, int height, int max_results, int *boxes, float *scores)
{
    Model *model = ((Handle *)handle)->model;
    std::vector<detect::anchor_point_stage_t> st;
    std::vector<std::pair<std::string, std::string>> nm;
    for (int i = 0; i < stages; i++) {
        st.push_back({strides[i], strides[i], strides[i] / 2, strides[i] / 2});
        nm.push_back({names[2 * i], names[2 * i + 1]});
    }
    detect::yolo11PostProcessor post(model, nullptr, score_thr, nms_thr, top_k, st);
    post.set_output_names(nm);
    if (post.postprocess() != ESP_OK)
        return -1;
    int k = 0;
    for (const detect::result_t &r : post.get_result(width, height, image)) {
        if (k >= max_results)
            break;
        boxes[5 * k] = r.category;
        for (int j = 0; j < 4; j++) boxes[5 * k + 1 + j] = r.box[j];
        scores[k++] = r.score;
    }
    return k;
}

/// dl::cls::ClsPostprocessor on the model's first output: up to `top_k` (category, score) pairs of image `image`,
/// best first.  Returns the number of results, -1 on error.
int espdl_model_classify(void *handle, int image, int top_k, float score_thr, int need_softmax, int *categories, float *scores)
{
    Model *model = ((Handle *)handle)->model;
    cls::ClsPostprocessor post(model, top_k, score_thr, need_softmax != 0);
    std::vector<cls::result_t> &r = post.postprocess(image);
    for (size_t i = 0; i < r.size(); i++) categories[i] = r[i].category, scores[i] = r[i].score;
    return (int)r.size();
}

/// dl::image::ImagePreprocessor over `n` host images [n][h][w][channels] (uint8) into the model's first input:
/// mean/std hold `channels` floats; crop = {x0, y0, x1, y1} or null; letterbox < 0 = off, else the background value.
int espdl_model_preprocess(void *handle, const unsigned char *images, int n, int h, int w, int channels, const float *mean, const float *stdv,
                           int rgb_swap, int letterbox_bg, const int *crop)
{
    Model *model = ((Handle *)handle)->model;
    image::ImagePreprocessor *pre = channels == 3
        ? new image::ImagePreprocessor(model, std::array<float, 3>{mean[0], mean[1], mean[2]}, std::array<float, 3>{stdv[0], stdv[1], stdv[2]}, rgb_swap != 0)
        : new image::ImagePreprocessor(model, mean[0], stdv[0]);
    if (letterbox_bg >= 0) {
        if (channels == 3)
            pre->enable_letterbox(std::array<uint8_t, 3>{(uint8_t)letterbox_bg, (uint8_t)letterbox_bg, (uint8_t)letterbox_bg});
        else
            pre->enable_letterbox((uint8_t)letterbox_bg);
    }
    std::vector<image::img_t> imgs;
    for (int i = 0; i < n; i++)
        imgs.push_back({(void *)(images + (size_t)i * h * w * channels), (uint16_t)w, (uint16_t)h,
                        channels == 3 ? image::DL_IMAGE_PIX_TYPE_RGB888 : image::DL_IMAGE_PIX_TYPE_GRAY});
    std::vector<int> crop_area;
    if (crop)
        crop_area.assign(crop, crop + 4);
    const esp_err_t e = pre->preprocess(imgs, crop_area);
    delete pre;
    return e == ESP_OK ? 0 : -1;
}

/// Text dump of what the C++ reader sees in a model file (no device needed): one line per node in execution
/// order "op_type<TAB>name<TAB>inputs<TAB>outputs", then one line per initializer "name<TAB>dtype<TAB>dims<TAB>n_exponents<TAB>sum".
const char *espdl_fbs_describe_key(const char *path, const unsigned char *key);
const char *espdl_fbs_describe(const char *path) { return espdl_fbs_describe_key(path, nullptr); }

/// PDL3 package check (no device needed): 1 = digest matches, 0 = it does not, -1 = not a PDL3 package.
/// `version16` (may be null) receives the version string, `package_size` (may be null) the header field.
int espdl_fbs_verify_package(const char *path, char *version16, unsigned *package_size)
{
    fbs::FbsLoader loader(path, fbs::MODEL_LOCATION_IN_SDCARD);
    if (!loader.is_pdl3())
        return -1;
    if (version16)
        loader.get_package_version(version16, 16);
    if (package_size)
        *package_size = loader.get_package_size();
    return loader.verify_package_sha256() ? 1 : 0;
}

/// As espdl_fbs_describe, with the 16-byte AES key of an encrypted model (null for a plain one).
const char *espdl_fbs_describe_key(const char *path, const unsigned char *key)
{
    static std::string text;
    text.clear();
    fbs::FbsLoader loader(path, fbs::MODEL_LOCATION_IN_SDCARD);
    fbs::FbsModel *m = loader.load(0, key, true);
    if (!m)
        return nullptr;
    text += "target\t" + m->get_model_metadata_prop("target") + "\n";
    for (const std::string &node : m->topological_sort()) {
        std::vector<std::string> ins, outs;
        m->get_operation_inputs_and_outputs(node, ins, outs);
        text += "node\t" + m->get_operation_type(node) + "\t" + node + "\t";
        for (auto &s : ins) text += s + ",";
        text += "\t";
        for (auto &s : outs) text += s + "," + vector_to_string(m->get_value_info_shape(s)) + "," + std::to_string(m->get_value_info_exponent(s)) + ";";
        std::vector<int> pads;
        if (m->get_operation_attribute(node, "pads", pads) == ESP_OK)
            text += "\tpads=" + vector_to_string(pads);
        std::string act;
        if (m->get_operation_attribute(node, "activation", act) == ESP_OK)
            text += "\tactivation=" + act;
        text += "\n";
        for (size_t i = 0; i < ins.size(); i++) {
            if (!m->is_parameter(ins[i]))
                continue;
            TensorBase *t = m->get_operation_parameter(node, (int)i);
            long long sum = 0;
            for (size_t b = 0; b < t->get_bytes(); b++) sum += ((const uint8_t *)t->data)[b];
            text += "param\t" + ins[i] + "\t" + std::to_string((int)t->dtype) + "\t" + vector_to_string(t->shape) + "\t" +
                std::to_string(t->exponent.size()) + "\t" + std::to_string(sum) + "\n";
            delete t;
        }
    }
    delete m;
    return text.c_str();
}

/// Runs the arena planner on a synthetic tensor list (no device needed).  Returns the arena size.
size_t espdl_plan_arena(int n, const int *first, const int *last, const size_t *bytes, const int *alias_of, size_t *offsets, int reuse)
{
    std::vector<TensorInfo> infos(n);
    for (int i = 0; i < n; i++) infos[i].first = first[i], infos[i].last = last[i], infos[i].bytes = bytes[i], infos[i].alias_of = alias_of[i];
    const size_t arena = MemoryManagerGreedy::plan(infos, reuse != 0);
    for (int i = 0; i < n; i++) offsets[i] = infos[i].offset;
    return arena;
}

/// The same with channel slices: tensor i with row_stride[i] != 0 lives view_offset[i] bytes into the buffer of alias_of[i].
size_t espdl_plan_arena_slices(int n, const int *first, const int *last, const size_t *bytes, const int *alias_of, const size_t *view_offset,
                               const int *row_stride, size_t *offsets, int reuse)
{
    std::vector<TensorInfo> infos(n);
    for (int i = 0; i < n; i++) {
        infos[i].first = first[i], infos[i].last = last[i], infos[i].bytes = bytes[i], infos[i].alias_of = alias_of[i];
        infos[i].view_offset = view_offset[i], infos[i].row_stride = row_stride[i];
    }
    const size_t arena = MemoryManagerGreedy::plan(infos, reuse != 0);
    for (int i = 0; i < n; i++) offsets[i] = infos[i].offset;
    return arena;
}

/// Per-module latency table as text: one "index<TAB>type<TAB>microseconds<TAB>name" line per module.
const char *espdl_model_profile(void *handle)
{
    Handle *h = (Handle *)handle;
    h->text.clear();
    for (auto &kv : h->model->get_module_info()) {
        char line[512];
        const size_t colon = kv.first.find(':');
        snprintf(line, sizeof(line), "%s\t%s\t%.2f\t%s\n", kv.first.substr(0, colon).c_str(), kv.second.type.c_str(), kv.second.latency_us,
                 kv.first.substr(colon + 1).c_str());
        h->text += line;
    }
    return h->text.c_str();
}

} // extern "C"
