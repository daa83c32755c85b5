#include "dl_module_ops.hpp"
#include "espdl_b200.h"

#include <climits>
#include <cassert>
#include <cmath>
#include <algorithm>
#include <cstring>

namespace dl {

ModelContext::~ModelContext()
{
    if (own_tensors)
        for (auto *t : m_variables) delete t;
}

int ModelContext::push_back_tensor(TensorBase *t, const std::string &name)
{
    m_variables.push_back(t);
    if (!name.empty())
        m_name2index[name] = (int)m_variables.size() - 1;
    return (int)m_variables.size() - 1;
}

TensorBase *ModelContext::get_tensor(const std::string &name)
{
    auto it = m_name2index.find(name);
    return it == m_name2index.end() ? nullptr : m_variables[it->second];
}

int ModelContext::get_tensor_index(const std::string &name)
{
    auto it = m_name2index.find(name);
    return it == m_name2index.end() ? -1 : it->second;
}

namespace module {

Module::Module(const char *n, module_inplace_t inplace, quant_type_t quant_type) : inplace(inplace), quant_type(quant_type)
{
    name = n ? strdup(n) : nullptr;
}

Module::~Module() { free(name); }

void Module::run(TensorBase *input, TensorBase *output, runtime_mode_t mode) { run(std::vector<TensorBase *>{input}, {output}, mode); }

void Module::run(std::vector<TensorBase *> inputs, std::vector<TensorBase *> outputs, runtime_mode_t mode)
{
    ModelContext context;
    m_inputs_index.clear();
    m_outputs_index.clear();
    for (auto *t : inputs) m_inputs_index.push_back(context.push_back_tensor(t));
    for (auto *t : outputs) m_outputs_index.push_back(context.push_back_tensor(t));
    prepare(&context);
    size_t ws = workspace_bytes(&context);
    if (ws && espdl_b200_arena_alloc(ws, &context.workspace) == ESPDL_OK)
        context.workspace_bytes = ws;
    forward(&context, mode);
    espdl_b200_stream_sync(nullptr);
    if (context.workspace)
        espdl_b200_arena_free(context.workspace);
}

static int espdl_dtype(TensorBase *t) { return (int)t->dtype; }
static int quant_dtype(quant_type_t q) { return q == QUANT_TYPE_SYMM_16BIT ? ESPDL_DTYPE_INT16 : ESPDL_DTYPE_INT8; }

// --------------------------------------------------------------------------------- Conv / Gemm
Conv::Conv(activation_type_t activation, std::vector<int> pads, std::vector<int> dilations, std::vector<int> strides, const char *name,
           const int group, quant_type_t quant_type, const std::string &target) :
    Module(name, MODULE_NON_INPLACE, quant_type), m_dilations(dilations), m_strides(strides), m_group(group), activation(activation),
    m_pads(pads), m_target(target)
{
    if (m_pads.empty())
        m_pads = {0, 0, 0, 0};
    if (m_strides.empty())
        m_strides = {1, 1};
    if (m_dilations.empty())
        m_dilations = {1, 1};
}

Conv::~Conv()
{
    for (void *p : {m_dev_exponents, m_grp_filter, m_grp_bias, m_grp_exponents})
        if (p)
            espdl_b200_arena_free(p);
    delete m_lut;
}

std::vector<std::vector<int>> Conv::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    // esp-dl/dl/module/include/dl_module_conv.hpp:81-102
    std::vector<int> in = input_shapes[0], f = input_shapes[1], out = in;
    if (in.size() == 3) { // conv1d: [N, W, C], filter [K, Cin, Cout]
        out[1] = (in[1] + m_pads[0] + m_pads[1] - m_dilations[0] * (f[0] - 1) - 1) / m_strides[0] + 1;
        out[2] = m_group == 1 ? f[2] : in[2];
    } else {
        out[1] = (in[1] + m_pads[0] + m_pads[1] - m_dilations[0] * (f[0] - 1) - 1) / m_strides[0] + 1;
        out[2] = (in[2] + m_pads[2] + m_pads[3] - m_dilations[1] * (f[1] - 1) - 1) / m_strides[1] + 1;
        out[3] = m_group == 1 ? f[3] : in[3];
    }
    return {out};
}

// Filter payloads are stored per export target although the declared shape is always [KH,KW,Cin,Cout]
// (esp-dl/dl/base/dl_base_conv2d.cpp:23-32,140-162; esp-dl/dl/base/dl_base.hpp:305-310,1255-1262):
//   "c"       dense [Cout][KH][KW][Cin], depthwise [KH][KW][C]
//   p4 / s3   dense [Cout/u][KH][KW][Cin][u] + tail [Cout%u][KH][KW][Cin]; depthwise [C/u][KH][KW][u] + tail [KH][KW][C%u]
// with u = 16 bytes / element size.  The kernels take the "c" order.
template <typename T> static void relayout_filter(T *data, int kh, int kw, int cin, int cout, bool depthwise)
{
    const int u = 16 / (int)sizeof(T);
    std::vector<T> src(data, data + (size_t)kh * kw * cin * (depthwise ? 1 : cout));
    if (!depthwise) {
        const int nb = cout / u;
        const size_t per = (size_t)kh * kw * cin;
        for (int o = 0; o < cout; o++)
            for (size_t r = 0; r < per; r++) {
                size_t s = o < nb * u ? ((size_t)(o / u) * per + r) * u + (o % u) : (size_t)nb * u * per + (size_t)(o - nb * u) * per + r;
                data[(size_t)o * per + r] = src[s];
            }
    } else {
        const int c = cin, nb = c / u, hw = kh * kw;
        for (int p = 0; p < hw; p++)
            for (int ch = 0; ch < c; ch++) {
                size_t s = ch < nb * u ? ((size_t)(ch / u) * hw + p) * u + (ch % u) : (size_t)nb * u * hw + (size_t)p * (c % u) + (ch - nb * u);
                data[(size_t)p * c + ch] = src[s];
            }
    }
}

esp_err_t Conv::prepare(ModelContext *context)
{
    if (m_prepared)
        return ESP_OK;
    m_prepared = true;
    TensorBase *filter = context->get_tensor(m_inputs_index[1]);
    if (!filter)
        return ESP_FAIL;
    std::vector<int> fs = filter->shape;
    if (fs.size() == 3)
        fs.insert(fs.begin(), 1); // conv1d filter [K, Cin, Cout] -> [1, K, Cin, Cout]
    if (fs.size() != 4)
        return ESP_FAIL;
    const bool dw = m_group != 1;
    if (m_target != "c" && !m_target.empty() && filter->data && !filter->device) {
        if (!filter->auto_free) {
            ESP_LOGE("Conv", "filter of %s aliases the model bytes; load with param_copy=true to re-order it", name ? name : "?");
            return ESP_FAIL;
        }
        if (filter->dtype == DATA_TYPE_INT8)
            relayout_filter((int8_t *)filter->data, fs[0], fs[1], fs[2], fs[3], dw);
        else if (filter->dtype == DATA_TYPE_INT16)
            relayout_filter((int16_t *)filter->data, fs[0], fs[1], fs[2], fs[3], dw);
    }
    if (filter->exponent.is_per_channel() && !m_dev_exponents) {
        std::vector<int32_t> e(filter->exponent.values().begin(), filter->exponent.values().end());
        if (espdl_b200_arena_alloc(e.size() * 4, &m_dev_exponents) != ESPDL_OK)
            return ESP_FAIL;
        if (espdl_b200_upload(m_dev_exponents, e.data(), e.size() * 4, nullptr) != ESPDL_OK || espdl_b200_stream_sync(nullptr) != ESPDL_OK)
            return ESP_FAIL;
    }
    for (size_t i = 1; i < m_inputs_index.size(); i++) {
        TensorBase *t = context->get_tensor(m_inputs_index[i]);
        if (t && !t->device && t->to_device() != ESP_OK)
            return ESP_FAIL;
    }
    if (m_lut && !m_lut->device && m_lut->to_device() != ESP_OK)
        return ESP_FAIL;
    // Pointwise int8 conv whose input rows are narrow: group g pixels so that a row has g * Cin channels.  Needed
    // when Cin is not a multiple of 16 (the tile kernel wants 16-byte rows) and wanted when Cin is small: the TMA
    // unit moves rows of 16-64 bytes at a fraction of HBM speed, rows of 128 bytes at full speed.  The widest
    // grouping whose block-diagonal filter stays small is used (ESPDL_B200_GROUP_K overrides the target width).
    TensorBase *input = context->get_tensor(m_inputs_index[0]);
    TensorBase *bias = has_bias() ? context->get_tensor(m_inputs_index[2]) : nullptr;
    if (!m_no_grouping && !m_gemm && !dw && input && input->shape.size() == 4 && quant_type == QUANT_TYPE_SYMM_8BIT && fs[0] == 1 && fs[1] == 1 &&
        m_strides[0] == 1 && m_strides[1] == 1 && m_pads[0] + m_pads[1] + m_pads[2] + m_pads[3] == 0 && filter->data &&
        !getenv("ESPDL_B200_NO_PIXEL_GROUPING")) {
        const int cin = fs[2], cout = fs[3];
        const long long pixels = (long long)input->shape[1] * input->shape[2];
        TensorBase *output = context->get_tensor(m_outputs_index[0]);
        const bool sliced = input->row_stride || (output && output->row_stride); // a slice has no runs of whole pixels
        m_group_px = sliced || m_lut_stride ? 1 : choose_pixel_group(cin, cout, pixels); // per-channel tables are indexed by the real channel
        if (m_group_px > 1) {
            const int g = m_group_px;
            std::vector<int8_t> wf((size_t)g * cout * g * cin, 0);
            const int8_t *w = (const int8_t *)filter->data; // [cout][cin]
            for (int blk = 0; blk < g; blk++)
                for (int o = 0; o < cout; o++)
                    memcpy(&wf[((size_t)(blk * cout + o) * g + blk) * cin], w + (size_t)o * cin, cin);
            std::vector<int32_t> bf, ef;
            for (int blk = 0; blk < g; blk++)
                for (int o = 0; o < cout; o++) {
                    if (bias && bias->data)
                        bf.push_back(((const int32_t *)bias->data)[o]);
                    ef.push_back(filter->exponent.get(filter->exponent.is_per_channel() ? o : 0));
                }
            bool ok = espdl_b200_arena_alloc(wf.size(), &m_grp_filter) == ESPDL_OK &&
                espdl_b200_upload(m_grp_filter, wf.data(), wf.size(), nullptr) == ESPDL_OK &&
                espdl_b200_arena_alloc(ef.size() * 4, &m_grp_exponents) == ESPDL_OK &&
                espdl_b200_upload(m_grp_exponents, ef.data(), ef.size() * 4, nullptr) == ESPDL_OK;
            if (ok && !bf.empty())
                ok = espdl_b200_arena_alloc(bf.size() * 4, &m_grp_bias) == ESPDL_OK &&
                    espdl_b200_upload(m_grp_bias, bf.data(), bf.size() * 4, nullptr) == ESPDL_OK;
            if (!ok || espdl_b200_stream_sync(nullptr) != ESPDL_OK)
                return ESP_FAIL;
        }
    }
    return espdl_b200_stream_sync(nullptr) == ESPDL_OK ? ESP_OK : ESP_FAIL;
}

int Conv::choose_pixel_group(int cin, int cout, long long pixels)
{
    // Score of a grouping g: input row width towards 128 bytes, output rows made of whole 16-byte groups and at
    // least 32 bytes wide, minus the extra L2 traffic of the g*g times larger filter (bytes per pixel relative to
    // the activations).  ESPDL_B200_GROUP_K, when set, caps g * Cin.
    const int cap = getenv("ESPDL_B200_GROUP_K") ? atoi(getenv("ESPDL_B200_GROUP_K")) : 1 << 20;
    int best = 1;
    double best_score = -1.0;
    for (int g : {1, 2, 4, 8, 16}) {
        if ((g * cin) % 16 != 0 || pixels % g != 0 || g * cout > 1024 || (g > 1 && g * cin > cap))
            continue;
        const double in_score = std::min(g * cin, 128) / 128.0;
        const double out_score = ((g * cout) % 16 == 0 ? 1.0 : 0.0) + 0.5 * std::min(g * cout, 32) / 32.0;
        const double filter_cost = g == 1 ? 0.0 : 0.5 * ((double)g * cin * cout / 128.0) / (cin + cout);
        const double score = in_score + out_score - filter_cost;
        if (score > best_score + 1e-9) {
            best_score = score;
            best = g;
        }
    }
    return best;
}

bool Conv::strided_ok(const std::vector<std::vector<int>> &in) const
{
    if (m_gemm || quant_type != QUANT_TYPE_SYMM_8BIT || in.size() < 2 || in[0].size() != 4 || in[1].size() != 4)
        return false;
    const std::vector<int> &x = in[0], &f = in[1];
    const int cin = x[3];
    if (m_group != 1)
        return cin % 16 == 0; // depthwise: both kernels take pixel strides
    const int cout = f[3];
    if (cin % 16 != 0 || cout % 16 != 0)
        return false;
    if (f[0] == 3 && f[1] == 3 && cin == 16)
        return false; // the banded kernel reads 128-byte runs of whole pixels
    const bool plain_1x1 = f[0] == 1 && f[1] == 1 && m_strides[0] == 1 && m_strides[1] == 1 && m_pads[0] + m_pads[1] + m_pads[2] + m_pads[3] == 0;
    if (plain_1x1 && !m_no_grouping && !getenv("ESPDL_B200_NO_PIXEL_GROUPING") && choose_pixel_group(cin, cout, (long long)x[1] * x[2]) != 1)
        return false;
    return true;
}

int Conv::fill_desc(ModelContext *context, void *desc)
{
    espdl_conv_desc &d = *(espdl_conv_desc *)desc;
    memset(&d, 0, sizeof(d));
    TensorBase *input = context->get_tensor(m_inputs_index[0]);
    TensorBase *filter = context->get_tensor(m_inputs_index[1]);
    TensorBase *bias = has_bias() ? context->get_tensor(m_inputs_index[2]) : nullptr;
    TensorBase *output = context->get_tensor(m_outputs_index[0]);
    if (!input || !filter || !output || !input->device || !filter->device || !output->device)
        return ESPDL_ERR_INVALID_ARG;
    d.input = input->device, d.filter = filter->device, d.bias = bias ? bias->device : nullptr, d.output = output->device;
    d.filter_exponents = (const int32_t *)m_dev_exponents;
    d.lut = m_lut ? (const int8_t *)m_lut->device : nullptr;
    d.lut_channel_stride = m_lut ? m_lut_stride : 0;
    d.dtype = quant_dtype(quant_type);
    std::vector<int> fs = filter->shape;
    if (m_gemm) {
        // esp-dl/dl/module/include/dl_module_gemm.hpp:96-99: every leading dim folds into rows
        const int k = input->shape.back();
        d.n = 1, d.in_h = 1, d.in_w = input->get_size() / k, d.in_c = k;
        d.out_h = 1, d.out_w = d.in_w, d.out_c = fs[3];
        d.kh = d.kw = 1, d.stride_h = d.stride_w = d.dilation_h = d.dilation_w = 1;
        d.group = 1;
    } else if (input->shape.size() == 4) {
        d.n = input->shape[0], d.in_h = input->shape[1], d.in_w = input->shape[2], d.in_c = input->shape[3];
        d.out_h = output->shape[1], d.out_w = output->shape[2], d.out_c = output->shape[3];
        d.kh = fs[0], d.kw = fs[1];
        d.stride_h = m_strides[0], d.stride_w = m_strides[1], d.dilation_h = m_dilations[0], d.dilation_w = m_dilations[1];
        d.pad_top = m_pads[0], d.pad_bottom = m_pads[1], d.pad_left = m_pads[2], d.pad_right = m_pads[3];
        d.group = m_group == 1 ? 1 : d.in_c;
    } else if (input->shape.size() == 3) { // conv1d: esp-dl/dl/base/dl_base.hpp:150-182
        d.n = input->shape[0], d.in_h = 1, d.in_w = input->shape[1], d.in_c = input->shape[2];
        d.out_h = 1, d.out_w = output->shape[1], d.out_c = output->shape[2];
        d.kh = 1, d.kw = fs[0];
        d.stride_h = 1, d.stride_w = m_strides[0], d.dilation_h = 1, d.dilation_w = m_dilations[0];
        d.pad_left = m_pads[0], d.pad_right = m_pads[1];
        d.group = m_group == 1 ? 1 : d.in_c;
    } else {
        return ESPDL_ERR_UNSUPPORTED;
    }
    d.in_exponent = input->exponent, d.out_exponent = m_lut ? m_pre_lut_exponent : (int)output->exponent;
    d.in_pixel_stride = input->row_stride, d.out_pixel_stride = output->row_stride; // channel slices (0 = dense)
    d.per_channel = filter->exponent.is_per_channel();
    d.filter_exponent = filter->exponent;
    if (m_group_px > 1) { // same bytes, g pixels per row: [N, 1, H*W/g, g*Cin] x block-diagonal filter -> [N, 1, H*W/g, g*Cout]
        const int g = m_group_px;
        d.in_w = d.in_h * d.in_w / g, d.in_h = 1, d.out_w = d.in_w, d.out_h = 1;
        d.in_c *= g, d.out_c *= g;
        d.filter = m_grp_filter, d.bias = m_grp_bias, d.filter_exponents = (const int32_t *)m_grp_exponents;
        d.per_channel = 1;
    }
    if (m_residual) {
        TensorBase *r = context->get_tensor(m_inputs_index.back());
        if (!r || !r->device)
            return ESPDL_ERR_INVALID_ARG;
        d.residual = r->device; // same NHWC memory as the output, also under pixel grouping
    }
    d.activation = activation == ReLU ? ESPDL_ACT_RELU : ESPDL_ACT_LINEAR;
    d.round_mode = context->round_mode;
    d.kernel = ESPDL_KERNEL_AUTO;
    if (activation != Linear && activation != ReLU)
        return ESPDL_ERR_UNSUPPORTED;
    return ESPDL_OK;
}

bool Conv::can_fold_add() const
{
    if (m_gemm || m_group != 1 || quant_type != QUANT_TYPE_SYMM_8BIT || m_lut)
        return false;
    for (int v : m_strides)
        if (v != 1)
            return false;
    for (int v : m_pads)
        if (v != 0)
            return false;
    for (int v : m_dilations)
        if (v != 1)
            return false;
    return activation == Linear || activation == ReLU;
}

bool Conv::is_pointwise() const { return can_fold_add(); }

bool Conv::is_dw3x3() const
{
    if (m_group == 1 || quant_type != QUANT_TYPE_SYMM_8BIT || m_lut || m_strides.size() != 2 || m_strides[0] != m_strides[1] ||
        (m_strides[0] != 1 && m_strides[0] != 2) || m_dilations[0] != 1 || m_dilations[1] != 1 || m_pads.size() != 4)
        return false;
    for (int v : m_pads)
        if (v < 0 || v > 1)
            return false;
    return activation == Linear || activation == ReLU;
}

// --------------------------------------------------------------------------------- FusedBlock
FusedBlock::FusedBlock(Conv *expand, Conv *dw, Conv *project, int e_expand, int e_dw, bool residual, const char *name) :
    Module(name, MODULE_NON_INPLACE, QUANT_TYPE_SYMM_8BIT), m_expand(expand), m_dw(dw), m_project(project), m_e_expand(e_expand), m_e_dw(e_dw),
    m_residual(residual)
{
}

FusedBlock::~FusedBlock()
{
    delete m_expand;
    delete m_dw;
    delete m_project;
}

// inputs: x, [expand filter, (bias)], dw filter, (bias), project filter, (bias), [residual]; a conv has a bias iff its
// module was given three inputs, which the fusion pass recorded in the conv's own index list
std::vector<std::vector<int>> FusedBlock::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    std::vector<int> cur = input_shapes[0];
    size_t at = 1;
    for (Conv *c : {m_expand, m_dw, m_project}) {
        if (!c)
            continue;
        const size_t n_params = c->m_inputs_index.size() - 1;
        std::vector<std::vector<int>> in = {cur, input_shapes[at]};
        cur = c->get_output_shape(in)[0];
        at += n_params;
    }
    return {cur};
}

esp_err_t FusedBlock::prepare(ModelContext *context)
{
    // hand every conv the context indices of its parameters (slot 0, its data input, is not used by Conv::prepare)
    size_t at = 1;
    for (Conv *c : {m_expand, m_dw, m_project}) {
        if (!c)
            continue;
        const size_t n_params = c->m_inputs_index.size() - 1;
        for (size_t i = 0; i < n_params; i++) c->m_inputs_index[1 + i] = m_inputs_index[at + i];
        c->m_inputs_index[0] = m_inputs_index[0];
        at += n_params;
        c->skip_pixel_grouping();
        if (c->prepare(context) != ESP_OK)
            return ESP_FAIL;
    }
    return ESP_OK;
}

void FusedBlock::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    espdl_block_desc d;
    memset(&d, 0, sizeof(d));
    TensorBase *x = context->get_tensor(m_inputs_index[0]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    int st = ESPDL_OK;
    if (!x || !out || !x->device || !out->device || x->shape.size() != 4) {
        st = ESPDL_ERR_INVALID_ARG;
    } else {
        auto stage = [&](Conv *c, const void *&filter, const void *&bias, const int32_t *&exps, int32_t &e_scalar, int32_t &act, int bit) {
            TensorBase *f = context->get_tensor(c->m_inputs_index[1]);
            TensorBase *b = c->has_bias() ? context->get_tensor(c->m_inputs_index[2]) : nullptr;
            filter = f->device, bias = b ? b->device : nullptr, exps = (const int32_t *)c->m_dev_exponents;
            e_scalar = f->exponent;
            if (f->exponent.is_per_channel())
                d.per_channel |= 1 << bit;
            act = c->activation == ReLU ? ESPDL_ACT_RELU : ESPDL_ACT_LINEAR;
            return f;
        };
        d.input = x->device, d.output = out->device;
        d.dtype = ESPDL_DTYPE_INT8;
        d.n = x->shape[0], d.in_h = x->shape[1], d.in_w = x->shape[2], d.in_c = x->shape[3];
        d.out_h = out->shape[1], d.out_w = out->shape[2], d.out_c = out->shape[3];
        d.hidden_c = d.in_c;
        if (m_expand) {
            TensorBase *f = stage(m_expand, d.expand_filter, d.expand_bias, d.expand_filter_exponents, d.expand_filter_exponent, d.expand_activation, 0);
            d.hidden_c = f->shape.back();
        }
        stage(m_dw, d.dw_filter, d.dw_bias, d.dw_filter_exponents, d.dw_filter_exponent, d.dw_activation, 1);
        stage(m_project, d.project_filter, d.project_bias, d.project_filter_exponents, d.project_filter_exponent, d.project_activation, 2);
        d.stride = m_dw->m_strides[0], d.pad_top = m_dw->m_pads[0], d.pad_left = m_dw->m_pads[2];
        d.in_exponent = x->exponent, d.expand_exponent = m_expand ? m_e_expand : (int)x->exponent, d.dw_exponent = m_e_dw, d.out_exponent = out->exponent;
        d.expand_clip_max = d.dw_clip_max = 127;
        d.round_mode = context->round_mode;
        if (m_residual) {
            TensorBase *r = context->get_tensor(m_inputs_index.back());
            if (!r || !r->device)
                st = ESPDL_ERR_INVALID_ARG;
            else
                d.residual = r->device;
        }
        if (st == ESPDL_OK)
            st = espdl_b200_fused_block(&d, context->stream);
    }
    if (st)
        ESP_LOGE("FusedBlock", "%s failed: %s %s", name ? name : "?", espdl_b200_strerror(st), espdl_b200_last_error());
    context->note(st);
}

size_t Conv::workspace_bytes(ModelContext *context)
{
    espdl_conv_desc d;
    size_t bytes = 0;
    if (fill_desc(context, &d) == ESPDL_OK)
        espdl_b200_conv2d_workspace_bytes(&d, &bytes);
    return bytes;
}

void Conv::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    espdl_conv_desc d;
    int st = fill_desc(context, &d);
    if (st == ESPDL_OK)
        st = espdl_b200_conv2d_ws(&d, context->workspace, context->workspace_bytes, context->stream);
    if (st)
        ESP_LOGE("Conv", "%s failed: %s %s", name ? name : "?", espdl_b200_strerror(st), espdl_b200_last_error());
    context->note(st);
}

static std::string model_target(fbs::FbsModel *m)
{
    std::string t = m->get_model_metadata_prop("target");
    if (t.empty()) {
        const char *env = getenv("ESPDL_B200_TARGET"); // exports without a target tag (the model zoo) are SIMD-layout files
        t = env ? env : "esp32p4";
    }
    return t;
}

Module *Conv::deserialize(fbs::FbsModel *fbs_model, std::string node_name)
{
    std::vector<int> pads, strides, dilations;
    int group = 1;
    activation_type_t activation_type = Linear;
    quant_type_t quant_type = QUANT_TYPE_NONE;
    fbs_model->get_operation_attribute(node_name, "pads", pads);
    fbs_model->get_operation_attribute(node_name, "strides", strides);
    fbs_model->get_operation_attribute(node_name, "dilations", dilations);
    fbs_model->get_operation_attribute(node_name, "group", group);
    fbs_model->get_operation_attribute(node_name, "activation", activation_type);
    fbs_model->get_operation_attribute(node_name, "quant_type", quant_type);
    if (quant_type != QUANT_TYPE_SYMM_8BIT && quant_type != QUANT_TYPE_SYMM_16BIT)
        return nullptr;
    if (pads.size() == 4)
        pads = {pads[0], pads[2], pads[1], pads[3]}; // ONNX [t,l,b,r] -> [t,b,l,r] (dl_module_conv.hpp:186-187)
    else if (pads.empty())
        pads = {0, 0, 0, 0};
    return new Conv(activation_type, pads, dilations, strides, node_name.c_str(), group, quant_type, model_target(fbs_model));
}

void Conv::print()
{
    ESP_LOGI("Conv", "pads %s strides %s dilations %s group %d activation %s quant %s", vector_to_string(m_pads).c_str(),
             vector_to_string(m_strides).c_str(), vector_to_string(m_dilations).c_str(), m_group, activation_type_to_string(activation),
             quant_type_to_string(quant_type));
}

Gemm::Gemm(activation_type_t activation, const char *name, quant_type_t quant_type, const std::string &target) :
    Conv(activation, {0, 0, 0, 0}, {1, 1}, {1, 1}, name, 1, quant_type, target)
{
    m_gemm = true;
}

std::vector<std::vector<int>> Gemm::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    std::vector<int> f = input_shapes[1];
    assert(f.size() == 4 && f[0] == 1 && f[1] == 1);
    assert(input_shapes[0].back() == f[2]);
    std::vector<int> out = input_shapes[0];
    out.back() = f[3];
    return {out};
}

Module *Gemm::deserialize(fbs::FbsModel *fbs_model, std::string node_name)
{
    activation_type_t activation_type = Linear;
    quant_type_t quant_type = QUANT_TYPE_NONE;
    int transA = -1, transB = -1;
    fbs_model->get_operation_attribute(node_name, "activation", activation_type);
    fbs_model->get_operation_attribute(node_name, "quant_type", quant_type);
    fbs_model->get_operation_attribute(node_name, "transA", transA);
    fbs_model->get_operation_attribute(node_name, "transB", transB);
    if ((transA != -1 && transA != 0) || (transB != -1 && transB != 0))
        return nullptr;
    if (quant_type != QUANT_TYPE_SYMM_8BIT && quant_type != QUANT_TYPE_SYMM_16BIT)
        return nullptr;
    return new Gemm(activation_type, node_name.c_str(), quant_type, model_target(fbs_model));
}

// --------------------------------------------------------------------------------- MatMul
static std::vector<int> broadcast_shape(const std::vector<int> &a, const std::vector<int> &b);

std::vector<std::vector<int>> MatMul::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    // torch.matmul shapes, as dl_module_matmul.hpp:48-113
    const std::vector<int> &a = input_shapes[0], &b = input_shapes[1];
    std::vector<int> out;
    if (a.size() == 1 && b.size() == 1) {
        out = {1};
    } else if (a.size() == 1) {
        out.assign(b.begin(), b.end() - 2);
        out.push_back(b.back());
    } else if (b.size() == 1) {
        out.assign(a.begin(), a.end() - 1);
    } else {
        const size_t n = std::max(a.size(), b.size());
        out = broadcast_shape(std::vector<int>(a.begin(), a.end() - 2), std::vector<int>(b.begin(), b.end() - 2));
        while (out.size() + 2 < n) out.insert(out.begin(), 1);
        out.push_back(a[a.size() - 2]);
        out.push_back(b.back());
    }
    return {out};
}

// Leading (batch) dims of both operands, right-aligned to the output's, and the matrix extents.
bool MatMul::slices(ModelContext *context, std::vector<int> &b0, std::vector<int> &b1, int &M, int &K, int &N)
{
    TensorBase *in0 = context->get_tensor(m_inputs_index[0]), *in1 = context->get_tensor(m_inputs_index[1]);
    if (!in0 || !in1 || in0->shape.empty() || in1->shape.empty() || in0->shape.size() > 4 || in1->shape.size() > 4)
        return false;
    const std::vector<int> &a = in0->shape, &b = in1->shape;
    K = a.back();
    M = a.size() == 1 ? 1 : a[a.size() - 2];
    N = b.size() == 1 ? 1 : b.back();
    if ((b.size() == 1 ? b[0] : b[b.size() - 2]) != K)
        return false;
    b0.assign(a.begin(), a.size() >= 2 ? a.end() - 2 : a.begin());
    b1.assign(b.begin(), b.size() >= 2 ? b.end() - 2 : b.begin());
    const size_t nb = std::max(b0.size(), b1.size());
    while (b0.size() < nb) b0.insert(b0.begin(), 1);
    while (b1.size() < nb) b1.insert(b1.begin(), 1);
    for (size_t i = 0; i < nb; i++)
        if (b0[i] != b1[i] && b0[i] != 1 && b1[i] != 1)
            return false;
    return true;
}

size_t MatMul::workspace_bytes(ModelContext *context)
{
    std::vector<int> b0, b1;
    int M, K, N;
    if (quant_type != QUANT_TYPE_SYMM_16BIT || !slices(context, b0, b1, M, K, N))
        return 0;
    espdl_conv_desc d;
    memset(&d, 0, sizeof(d));
    d.dtype = ESPDL_DTYPE_INT16, d.n = 1, d.in_h = d.out_h = 1, d.in_w = d.out_w = M, d.in_c = K, d.out_c = N, d.kh = d.kw = 1;
    d.stride_h = d.stride_w = d.dilation_h = d.dilation_w = 1, d.group = 1;
    // the query validates the descriptor like a launch does, so it needs the operands' addresses too
    TensorBase *in0 = context->get_tensor(m_inputs_index[0]), *in1 = context->get_tensor(m_inputs_index[1]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    if (!in0 || !in1 || !out || !in0->device || !in1->device || !out->device)
        return 0;
    d.input = in0->device, d.filter = in1->device, d.output = out->device;
    // the batched form (one launch over all slices) splits all rows at once
    long long count = 1;
    for (size_t i = 0; i < b0.size(); i++) count *= std::max(b0[i], b1[i]);
    bool shared = true;
    for (int v : b1) shared = shared && v == 1;
    if (shared && count > 1 && count <= 0x7fffffffll)
        d.n = (int)count;
    size_t bytes = 0;
    return espdl_b200_conv2d_workspace_bytes(&d, &bytes) == ESPDL_OK ? bytes : 0;
}

esp_err_t MatMul::prepare(ModelContext *context)
{
    for (int idx : m_inputs_index) {
        TensorBase *t = context->get_tensor(idx);
        if (t && t->data && !t->device && t->to_device() != ESP_OK) // host data and no device copy: a parameter
            return ESP_FAIL;
    }
    return espdl_b200_stream_sync(nullptr) == ESPDL_OK ? ESP_OK : ESP_FAIL;
}

void MatMul::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *in0 = context->get_tensor(m_inputs_index[0]), *in1 = context->get_tensor(m_inputs_index[1]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    std::vector<int> b0, b1;
    int M = 0, K = 0, N = 0, st = ESPDL_OK;
    if (!in0 || !in1 || !out || !in0->device || !in1->device || !out->device || !slices(context, b0, b1, M, K, N)) {
        context->note(ESPDL_ERR_INVALID_ARG);
        return;
    }
    const size_t es = quant_type == QUANT_TYPE_SYMM_16BIT ? 2 : 1;
    // one Gemm per batch slice, the operand with extent 1 in a batch dim is reused (dl_module_matmul.hpp:191-520)
    std::vector<int> ob(b0.size());
    long long count = 1;
    for (size_t i = 0; i < b0.size(); i++) {
        ob[i] = std::max(b0[i], b1[i]);
        count *= ob[i];
    }
    // all slices in one launch when the batch dims need no index arithmetic: both operands carry every slice (the
    // filter then steps K*N per slice), or input1 is one matrix shared by all slices (a plain Gemm over all rows)
    bool full0 = true, full1 = true, none1 = true;
    for (size_t i = 0; i < ob.size(); i++) {
        full0 = full0 && b0[i] == ob[i];
        full1 = full1 && b1[i] == ob[i];
        none1 = none1 && b1[i] == 1;
    }
    if (count > 1 && full0 && (full1 || none1) && count <= 0x7fffffffll && (long long)K * N <= 0x7fffffffll) {
        espdl_conv_desc d;
        memset(&d, 0, sizeof(d));
        d.input = in0->device, d.filter = in1->device, d.output = out->device;
        d.dtype = quant_dtype(quant_type);
        d.n = (int)count, d.in_h = d.out_h = 1, d.in_w = d.out_w = M, d.in_c = K, d.out_c = N, d.kh = d.kw = 1;
        d.stride_h = d.stride_w = d.dilation_h = d.dilation_w = 1, d.group = 1;
        d.filter_image_stride = none1 ? 0 : K * N;
        d.in_exponent = in0->exponent, d.out_exponent = out->exponent, d.filter_exponent = in1->exponent, d.per_channel = 0;
        d.activation = m_activation == ReLU ? ESPDL_ACT_RELU : ESPDL_ACT_LINEAR;
        d.round_mode = context->round_mode;
        st = espdl_b200_conv2d_ws(&d, context->workspace, context->workspace_bytes, context->stream);
        count = 0; // nothing left for the per-slice loop
    }
    for (long long s = 0; s < count && !st; s++) {
        long long rem = s, i0 = 0, i1 = 0, m0 = 1, m1 = 1;
        for (int i = (int)ob.size() - 1; i >= 0; i--) {
            const int idx = (int)(rem % ob[i]);
            rem /= ob[i];
            i0 += (b0[i] == 1 ? 0 : idx) * m0;
            i1 += (b1[i] == 1 ? 0 : idx) * m1;
            m0 *= b0[i];
            m1 *= b1[i];
        }
        espdl_conv_desc d;
        memset(&d, 0, sizeof(d));
        d.input = (const char *)in0->device + (size_t)i0 * M * K * es;
        d.filter = (const char *)in1->device + (size_t)i1 * K * N * es; // read as [N][K], as the reference's conv kernel does
        d.output = (char *)out->device + (size_t)s * M * N * es;
        d.dtype = quant_dtype(quant_type);
        d.n = 1, d.in_h = d.out_h = 1, d.in_w = d.out_w = M, d.in_c = K, d.out_c = N, d.kh = d.kw = 1;
        d.stride_h = d.stride_w = d.dilation_h = d.dilation_w = 1, d.group = 1;
        d.in_exponent = in0->exponent, d.out_exponent = out->exponent, d.filter_exponent = in1->exponent, d.per_channel = 0;
        d.activation = m_activation == ReLU ? ESPDL_ACT_RELU : ESPDL_ACT_LINEAR;
        d.round_mode = context->round_mode;
        st = espdl_b200_conv2d_ws(&d, context->workspace, context->workspace_bytes, context->stream);
    }
    if (st)
        ESP_LOGE("MatMul", "%s failed: %s %s", name ? name : "?", espdl_b200_strerror(st), espdl_b200_last_error());
    context->note(st);
}

Module *MatMul::deserialize(fbs::FbsModel *fbs_model, std::string node_name)
{
    activation_type_t activation_type = Linear;
    quant_type_t quant_type = QUANT_TYPE_NONE;
    fbs_model->get_operation_attribute(node_name, "activation", activation_type);
    fbs_model->get_operation_attribute(node_name, "quant_type", quant_type);
    if (quant_type != QUANT_TYPE_SYMM_8BIT && quant_type != QUANT_TYPE_SYMM_16BIT)
        return nullptr;
    if (activation_type != Linear && activation_type != ReLU)
        return nullptr;
    return new MatMul(activation_type, node_name.c_str(), quant_type);
}

// --------------------------------------------------------------------------------- elementwise
static std::vector<int> broadcast_shape(const std::vector<int> &a, const std::vector<int> &b)
{
    const size_t n = std::max(a.size(), b.size());
    std::vector<int> out(n);
    for (size_t i = 0; i < n; i++) {
        const int da = i < n - a.size() ? 1 : a[i - (n - a.size())];
        const int db = i < n - b.size() ? 1 : b[i - (n - b.size())];
        out[i] = std::max(da, db);
    }
    return out;
}

std::vector<std::vector<int>> Elementwise::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    return {broadcast_shape(input_shapes[0], input_shapes[1])};
}

// Shapes with more than four axes are merged from the right where both operands are dense.
static bool pack_shapes(const std::vector<int> &out, const std::vector<int> &a, const std::vector<int> &b, espdl_eltwise_desc &d)
{
    const size_t n = out.size();
    std::vector<int> o(out), x(n, 1), y(n, 1);
    for (size_t i = 0; i < a.size(); i++) x[n - a.size() + i] = a[i];
    for (size_t i = 0; i < b.size(); i++) y[n - b.size() + i] = b[i];
    // drop unit axes, then merge neighbours on which both operands broadcast the same way
    std::vector<int> mo, mx, my;
    for (size_t i = 0; i < n; i++) {
        if (o[i] == 1)
            continue;
        const bool fx = x[i] == o[i], fy = y[i] == o[i];
        if (!mo.empty() && (mx.back() == mo.back()) == fx && (my.back() == mo.back()) == fy) {
            mo.back() *= o[i], mx.back() *= x[i], my.back() *= y[i];
        } else {
            mo.push_back(o[i]), mx.push_back(x[i]), my.push_back(y[i]);
        }
    }
    if (mo.empty())
        mo = {1}, mx = {1}, my = {1};
    if (mo.size() > 4)
        return false;
    d.ndim = (int)mo.size();
    for (size_t i = 0; i < mo.size(); i++) d.out_shape[i] = mo[i], d.in0_shape[i] = mx[i], d.in1_shape[i] = my[i];
    return true;
}

esp_err_t Elementwise::prepare(ModelContext *context)
{
    for (int idx : m_inputs_index) {
        TensorBase *t = context->get_tensor(idx);
        if (t && t->data && !t->device && t->to_device() != ESP_OK) // host data and no device copy: a parameter
            return ESP_FAIL;
    }
    return espdl_b200_stream_sync(nullptr) == ESPDL_OK ? ESP_OK : ESP_FAIL;
}

void Elementwise::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *a = context->get_tensor(m_inputs_index[0]), *b = context->get_tensor(m_inputs_index[1]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    espdl_eltwise_desc d;
    memset(&d, 0, sizeof(d));
    int st = ESPDL_OK;
    if (!a || !b || !out || !a->device || !b->device || !out->device)
        st = ESPDL_ERR_INVALID_ARG;
    const bool sliced = !st && (a->row_stride || b->row_stride || out->row_stride);
    if (sliced) { // operands of one shape: rows of the last axis, each tensor with its own row stride
        if (a->shape != out->shape || b->shape != out->shape) {
            st = ESPDL_ERR_UNSUPPORTED;
        } else {
            const int c = out->shape.back();
            d.ndim = 2;
            d.out_shape[0] = d.in0_shape[0] = d.in1_shape[0] = out->get_size() / c;
            d.out_shape[1] = d.in0_shape[1] = d.in1_shape[1] = c;
            d.in0_row_stride = a->row_stride, d.in1_row_stride = b->row_stride, d.out_row_stride = out->row_stride;
        }
    } else if (!st && !pack_shapes(out->shape, a->shape, b->shape, d)) {
        st = ESPDL_ERR_UNSUPPORTED;
    }
    if (!st) {
        d.input0 = a->device, d.input1 = b->device, d.output = out->device;
        d.op = m_op, d.in_dtype = espdl_dtype(a), d.out_dtype = espdl_dtype(out);
        d.in0_exponent = a->exponent, d.in1_exponent = b->exponent, d.out_exponent = out->exponent;
        d.round_mode = context->round_mode;
        st = espdl_b200_eltwise(&d, context->stream);
    }
    if (st)
        ESP_LOGE("Elementwise", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

bool Elementwise::same_shapes(const std::vector<std::vector<int>> &in) const
{
    return m_op != ESPDL_ELT_DIV && in.size() == 2 && !in[0].empty() && in[0] == in[1];
}

Add::Add(const char *name, module_inplace_t inplace, quant_type_t quant_type) : Elementwise(ESPDL_ELT_ADD, name, inplace, quant_type) {}
Sub::Sub(const char *name, module_inplace_t inplace, quant_type_t quant_type) : Elementwise(ESPDL_ELT_SUB, name, inplace, quant_type) {}
Mul::Mul(const char *name, module_inplace_t inplace, quant_type_t quant_type) : Elementwise(ESPDL_ELT_MUL, name, inplace, quant_type) {}

static quant_type_t node_quant(fbs::FbsModel *m, const std::string &node)
{
    quant_type_t q = QUANT_TYPE_NONE;
    m->get_operation_attribute(node, "quant_type", q);
    return q;
}

Module *Add::deserialize(fbs::FbsModel *m, std::string node) { return new Add(node.c_str(), MODULE_INPLACE_CHANGED_BUFFER, node_quant(m, node)); }
Module *Sub::deserialize(fbs::FbsModel *m, std::string node) { return new Sub(node.c_str(), MODULE_INPLACE_CHANGED_BUFFER, node_quant(m, node)); }
Module *Mul::deserialize(fbs::FbsModel *m, std::string node) { return new Mul(node.c_str(), MODULE_INPLACE_CHANGED_BUFFER, node_quant(m, node)); }

#define ESPDL_B200_TWO_OPERAND_MODULE(NAME, OP)                                                                                  \
    NAME::NAME(const char *name, module_inplace_t inplace, quant_type_t quant_type) : Elementwise(OP, name, inplace, quant_type) {} \
    Module *NAME::deserialize(fbs::FbsModel *m, std::string node) { return new NAME(node.c_str(), MODULE_INPLACE_CHANGED_BUFFER, node_quant(m, node)); }
ESPDL_B200_TWO_OPERAND_MODULE(Max, ESPDL_ELT_MAX)
ESPDL_B200_TWO_OPERAND_MODULE(Min, ESPDL_ELT_MIN)
ESPDL_B200_TWO_OPERAND_MODULE(Div, ESPDL_ELT_DIV)
ESPDL_B200_TWO_OPERAND_MODULE(Mod, ESPDL_ELT_MOD)
ESPDL_B200_TWO_OPERAND_MODULE(Greater, ESPDL_ELT_GREATER)
ESPDL_B200_TWO_OPERAND_MODULE(GreaterOrEqual, ESPDL_ELT_GREATER_EQUAL)
ESPDL_B200_TWO_OPERAND_MODULE(Equal, ESPDL_ELT_EQUAL)
ESPDL_B200_TWO_OPERAND_MODULE(Less, ESPDL_ELT_LESS)
ESPDL_B200_TWO_OPERAND_MODULE(LessOrEqual, ESPDL_ELT_LESS_EQUAL)
#undef ESPDL_B200_TWO_OPERAND_MODULE

esp_err_t Unary::prepare(ModelContext *context)
{
    (void)context;
    if (m_param && !m_param->device) {
        if (m_param->to_device() != ESP_OK || espdl_b200_stream_sync(nullptr) != ESPDL_OK)
            return ESP_FAIL;
    }
    return ESP_OK;
}

void Unary::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *in = context->get_tensor(m_inputs_index[0]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    espdl_eltwise_desc d;
    memset(&d, 0, sizeof(d));
    int st = ESPDL_OK;
    if (!in || !out || !in->device || !out->device)
        st = ESPDL_ERR_INVALID_ARG;
    if (!st) {
        d.input0 = in->device, d.output = out->device;
        d.input1 = m_param ? m_param->device : nullptr;
        d.op = m_op, d.in_dtype = espdl_dtype(in), d.out_dtype = espdl_dtype(out);
        d.in0_exponent = in->exponent, d.out_exponent = out->exponent;
        d.in1_exponent = m_param ? (int)m_param->exponent : 0;
        d.clip_lo = m_clip_lo, d.clip_hi = m_clip_hi;
        d.round_mode = context->round_mode;
        if (m_op == ESPDL_ELT_LUT && in->dtype == DATA_TYPE_INT16 && m_param && m_param->get_size() > 1) {
            // step = 65536 / (entries - 1), a power of two (dl_module_lut.hpp:33-36, :64-67)
            int step = 65536 / (m_param->get_size() - 1);
            while (step > 1) d.lut_shift++, step >>= 1;
        }
        if (in->row_stride || out->row_stride) { // a channel slice on either side: rows of the last axis
            const int c = in->shape.back();
            d.ndim = 2;
            d.out_shape[0] = d.in0_shape[0] = in->get_size() / c, d.out_shape[1] = d.in0_shape[1] = c;
            d.in1_shape[0] = d.in1_shape[1] = 1;
            d.in0_row_stride = in->row_stride, d.out_row_stride = out->row_stride;
            if (m_op == ESPDL_ELT_PRELU)
                st = ESPDL_ERR_UNSUPPORTED;
        } else if (m_op == ESPDL_ELT_PRELU && in->shape.size() <= 4) {
            d.ndim = (int)in->shape.size();
            for (int i = 0; i < d.ndim; i++) d.out_shape[i] = d.in0_shape[i] = in->shape[i], d.in1_shape[i] = 1;
        } else {
            d.ndim = 1;
            d.out_shape[0] = d.in0_shape[0] = in->get_size();
            d.in1_shape[0] = 1;
        }
        if (!st)
            st = espdl_b200_eltwise(&d, context->stream);
    }
    if (st)
        ESP_LOGE("Unary", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

bool Unary::strided_input_ok(int i, const std::vector<std::vector<int>> &in) const
{
    return i == 0 && m_op != ESPDL_ELT_PRELU && !in.empty() && !in[0].empty();
}

RequantizeLinear::RequantizeLinear(const char *name, module_inplace_t inplace, quant_type_t quant_type) :
    Unary(ESPDL_ELT_REQUANTIZE, name, inplace, quant_type)
{
}
Module *RequantizeLinear::deserialize(fbs::FbsModel *m, std::string node)
{
    return new RequantizeLinear(node.c_str(), MODULE_INPLACE_CHANGED_BUFFER, node_quant(m, node));
}

LUT::LUT(const char *name, TensorBase *table, module_inplace_t inplace, quant_type_t quant_type) :
    Unary(ESPDL_ELT_LUT, name, inplace, quant_type, table)
{
}
// LUT nodes and every activation exported with a `lut` attribute (Swish, Sigmoid, Tanh, HardSwish, Gelu, ...)
// (esp-dl/dl/module/include/dl_module_swish.hpp:84-103).
Module *LUT::deserialize(fbs::FbsModel *m, std::string node)
{
    quant_type_t q = node_quant(m, node);
    if (q != QUANT_TYPE_SYMM_8BIT && q != QUANT_TYPE_SYMM_16BIT)
        return nullptr; // the float fall-backs are not on this path
    TensorBase *table = m->get_operation_lut(node);
    if (!table)
        return nullptr;
    if (!table->auto_free) { // own a private copy: the module uploads and frees it
        TensorBase *copy = new TensorBase(table->shape, table->data, (int)table->exponent, table->dtype, true);
        delete table;
        table = copy;
    }
    return new LUT(node.c_str(), table, MODULE_INPLACE_CHANGED_BUFFER, q);
}

Clip::Clip(const char *name, module_inplace_t inplace, quant_type_t quant_type) : Unary(ESPDL_ELT_CLIP, name, inplace, quant_type) {}

void Clip::forward(ModelContext *context, runtime_mode_t mode)
{
    // min / max are one-element initializers in the input's quantised scale (dl_module_clip.hpp:78-90)
    const bool s16 = quant_type == QUANT_TYPE_SYMM_16BIT;
    m_clip_lo = s16 ? -32768 : -128, m_clip_hi = s16 ? 32767 : 127;
    auto scalar = [&](size_t idx, int &dst) {
        if (m_inputs_index.size() > idx) {
            TensorBase *t = context->get_tensor(m_inputs_index[idx]);
            if (t && t->data)
                dst = t->dtype == DATA_TYPE_INT16 ? (int)((int16_t *)t->data)[0] : (int)((int8_t *)t->data)[0];
        }
    };
    scalar(1, m_clip_lo);
    scalar(2, m_clip_hi);
    Unary::forward(context, mode);
}

Module *Clip::deserialize(fbs::FbsModel *m, std::string node)
{
    quant_type_t q = node_quant(m, node);
    if (q == QUANT_TYPE_SYMM_8BIT) {
        Module *lut = LUT::deserialize(m, node);
        if (lut)
            return lut;
    }
    return new Clip(node.c_str(), MODULE_INPLACE_CHANGED_BUFFER, q);
}

Relu::Relu(const char *name, module_inplace_t inplace, quant_type_t quant_type) : Unary(ESPDL_ELT_RELU, name, inplace, quant_type) {}
Module *Relu::deserialize(fbs::FbsModel *m, std::string node)
{
    quant_type_t q = node_quant(m, node);
    if (q == QUANT_TYPE_SYMM_8BIT) {
        Module *lut = LUT::deserialize(m, node);
        if (lut)
            return lut;
    }
    return new Relu(node.c_str(), MODULE_INPLACE_CHANGED_BUFFER, q);
}

PRelu::PRelu(const char *name, TensorBase *alpha, module_inplace_t inplace, quant_type_t quant_type) :
    Unary(ESPDL_ELT_PRELU, name, inplace, quant_type, alpha)
{
}
Module *PRelu::deserialize(fbs::FbsModel *m, std::string node)
{
    quant_type_t q = node_quant(m, node);
    if (q == QUANT_TYPE_SYMM_8BIT) {
        Module *lut = LUT::deserialize(m, node);
        if (lut)
            return lut;
    }
    TensorBase *alpha = m->get_operation_parameter(node, 1);
    if (!alpha)
        return nullptr;
    if (!alpha->auto_free) {
        TensorBase *copy = new TensorBase(alpha->shape, alpha->data, (int)alpha->exponent, alpha->dtype, true);
        delete alpha;
        alpha = copy;
    }
    return new PRelu(node.c_str(), alpha, MODULE_INPLACE_CHANGED_BUFFER, q);
}

// --------------------------------------------------------------------------------- pooling
std::vector<std::vector<int>> Pool::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    std::vector<int> in = input_shapes[0], out = in;
    if (m_op == ESPDL_POOL_GLOBAL_AVG) {
        for (size_t i = 1; i + 1 < out.size(); i++) out[i] = 1; // keeps dim 0 (the reference hard-codes 1 there)
        return {out};
    }
    if (in.size() == 4) {
        out[1] = (in[1] + m_pads[0] + m_pads[1] - m_kernel[0]) / m_strides[0] + 1;
        out[2] = (in[2] + m_pads[2] + m_pads[3] - m_kernel[1]) / m_strides[1] + 1;
    } else {
        out[1] = (in[1] + m_pads[0] + m_pads[1] - m_kernel[0]) / m_strides[0] + 1;
    }
    return {out};
}

void Pool::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *in = context->get_tensor(m_inputs_index[0]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    espdl_pool_desc d;
    memset(&d, 0, sizeof(d));
    int st = (!in || !out || !in->device || !out->device) ? ESPDL_ERR_INVALID_ARG : ESPDL_OK;
    if (!st) {
        d.input = in->device, d.output = out->device, d.op = m_op, d.dtype = quant_dtype(quant_type);
        if (in->shape.size() == 4) {
            d.n = in->shape[0], d.in_h = in->shape[1], d.in_w = in->shape[2], d.c = in->shape[3];
            d.out_h = out->shape[1], d.out_w = out->shape[2];
            if (m_op != ESPDL_POOL_GLOBAL_AVG) {
                d.kh = m_kernel[0], d.kw = m_kernel[1], d.stride_h = m_strides[0], d.stride_w = m_strides[1];
                d.pad_top = m_pads[0], d.pad_bottom = m_pads[1], d.pad_left = m_pads[2], d.pad_right = m_pads[3];
            }
        } else if (in->shape.size() == 3) {
            d.n = in->shape[0], d.in_h = 1, d.in_w = in->shape[1], d.c = in->shape[2];
            d.out_h = 1, d.out_w = out->shape[1];
            if (m_op != ESPDL_POOL_GLOBAL_AVG) {
                d.kh = 1, d.kw = m_kernel[0], d.stride_h = 1, d.stride_w = m_strides[0];
                d.pad_left = m_pads[0], d.pad_right = m_pads[1];
            }
        } else {
            st = ESPDL_ERR_UNSUPPORTED;
        }
        d.in_exponent = in->exponent, d.out_exponent = out->exponent;
        if (!st)
            st = espdl_b200_pool(&d, context->stream);
    }
    if (st)
        ESP_LOGE("Pool", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

static void pool_attrs(fbs::FbsModel *m, const std::string &node, std::vector<int> &k, std::vector<int> &p, std::vector<int> &s)
{
    m->get_operation_attribute(node, "kernel_shape", k);
    m->get_operation_attribute(node, "pads", p);
    m->get_operation_attribute(node, "strides", s);
    if (p.size() == 4)
        p = {p[0], p[2], p[1], p[3]};
    else if (p.empty())
        p = std::vector<int>(k.size() * 2, 0);
    if (s.empty())
        s = std::vector<int>(k.size(), 1);
}

MaxPool::MaxPool(const char *name, const std::vector<int> &filter_shape, const std::vector<int> &padding, const std::vector<int> &strides,
                 quant_type_t quant_type) :
    Pool(ESPDL_POOL_MAX, name, filter_shape, padding.empty() ? std::vector<int>(filter_shape.size() * 2, 0) : padding, strides, quant_type)
{
}
Module *MaxPool::deserialize(fbs::FbsModel *m, std::string node)
{
    std::vector<int> k, p, s;
    pool_attrs(m, node, k, p, s);
    quant_type_t q = node_quant(m, node);
    if (q != QUANT_TYPE_SYMM_8BIT && q != QUANT_TYPE_SYMM_16BIT)
        return nullptr;
    return new MaxPool(node.c_str(), k, p, s, q);
}
AveragePool::AveragePool(const char *name, const std::vector<int> &kernel_shape, const std::vector<int> &pads,
                         const std::vector<int> &strides, quant_type_t quant_type) :
    Pool(ESPDL_POOL_AVG, name, kernel_shape, pads.empty() ? std::vector<int>(kernel_shape.size() * 2, 0) : pads, strides, quant_type)
{
}
Module *AveragePool::deserialize(fbs::FbsModel *m, std::string node)
{
    std::vector<int> k, p, s;
    pool_attrs(m, node, k, p, s);
    quant_type_t q = node_quant(m, node);
    if (q != QUANT_TYPE_SYMM_8BIT && q != QUANT_TYPE_SYMM_16BIT)
        return nullptr;
    return new AveragePool(node.c_str(), k, p, s, q);
}
GlobalAveragePool::GlobalAveragePool(const char *name, quant_type_t quant_type) : Pool(ESPDL_POOL_GLOBAL_AVG, name, {}, {}, {}, quant_type) {}
Module *GlobalAveragePool::deserialize(fbs::FbsModel *m, std::string node)
{
    quant_type_t q = node_quant(m, node);
    if (q != QUANT_TYPE_SYMM_8BIT && q != QUANT_TYPE_SYMM_16BIT)
        return nullptr;
    return new GlobalAveragePool(node.c_str(), q);
}

// --------------------------------------------------------------------------------- resize
Resize::Resize(const char *name, const resize_mode_t resize_mode, const std::vector<float> scales, const std::vector<int64_t> sizes,
               const bool align_corners, quant_type_t quant_type) :
    Module(name, MODULE_NON_INPLACE, quant_type), m_resize_mode(resize_mode), m_scales(scales), m_sizes(sizes),
    m_align_corners(align_corners)
{
}

std::vector<std::vector<int>> Resize::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    // scales / sizes are given in NCHW order (dl_module_resize.hpp:55-81)
    std::vector<int> in = input_shapes[0], out = in;
    if (m_scales.empty() && m_sizes.size() == in.size()) {
        m_scales.assign(in.size(), 1.f);
        if (in.size() == 4) {
            m_scales[2] = (float)m_sizes[2] / in[1];
            m_scales[3] = (float)m_sizes[3] / in[2];
        } else {
            m_scales[2] = (float)m_sizes[2] / in[1];
        }
    }
    if (in.size() == 4) {
        out[1] = (int)(in[1] * m_scales[2]);
        out[2] = (int)(in[2] * m_scales[3]);
    } else if (in.size() == 3) {
        out[1] = (int)(in[1] * m_scales[2]);
    }
    return {out};
}

void Resize::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *in = context->get_tensor(m_inputs_index[0]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    espdl_resize_desc d;
    memset(&d, 0, sizeof(d));
    int st = (!in || !out || !in->device || !out->device) ? ESPDL_ERR_INVALID_ARG : ESPDL_OK;
    if (!st && m_resize_mode != RESIZE_NEAREST && m_resize_mode != RESIZE_LINEAR)
        st = ESPDL_ERR_UNSUPPORTED;
    if (!st) {
        d.input = in->device, d.output = out->device, d.dtype = quant_dtype(quant_type);
        if (in->shape.size() == 4) {
            d.n = in->shape[0], d.in_h = in->shape[1], d.in_w = in->shape[2], d.c = in->shape[3];
            d.out_h = out->shape[1], d.out_w = out->shape[2];
            d.scale_h = m_scales[2], d.scale_w = m_scales[3];
        } else {
            d.n = in->shape[0], d.in_h = 1, d.in_w = in->shape[1], d.c = in->shape[2];
            d.out_h = 1, d.out_w = out->shape[1];
            d.scale_h = 1, d.scale_w = m_scales[2];
        }
        d.in_exponent = in->exponent, d.out_exponent = out->exponent;
        d.out_pixel_stride = out->row_stride;
        d.mode = m_resize_mode == RESIZE_NEAREST ? 0 : (m_align_corners ? 2 : 1);
        st = espdl_b200_resize(&d, context->stream);
    }
    if (st)
        ESP_LOGE("Resize", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

Module *Resize::deserialize(fbs::FbsModel *m, std::string node)
{
    quant_type_t q = node_quant(m, node);
    resize_mode_t mode = RESIZE_NEAREST;
    std::string ctm;
    m->get_operation_attribute(node, "mode", mode);
    m->get_operation_attribute(node, "coordinate_transformation_mode", ctm);
    std::vector<float> scales;
    std::vector<int64_t> sizes;
    if (TensorBase *t = m->get_operation_parameter(node, 2)) {
        scales.assign((float *)t->data, (float *)t->data + t->get_size());
        delete t;
    }
    if (TensorBase *t = m->get_operation_parameter(node, 3)) {
        sizes.assign((int64_t *)t->data, (int64_t *)t->data + t->get_size());
        delete t;
    }
    if (q != QUANT_TYPE_SYMM_8BIT && q != QUANT_TYPE_SYMM_16BIT)
        return nullptr;
    return new Resize(node.c_str(), mode, scales, sizes, ctm == "align_corners", q);
}

// --------------------------------------------------------------------------------- data movement
static int enqueue_copy(ModelContext *ctx, const void *src, void *dst, int es, const std::vector<int> &shape,
                        const std::vector<long long> &ss, const std::vector<long long> &ds)
{
    // merge to at most six axes from the right where both sides are contiguous
    std::vector<int> sh;
    std::vector<long long> s, t;
    for (size_t i = 0; i < shape.size(); i++) {
        if (shape[i] == 1)
            continue;
        if (!sh.empty() && s.back() == ss[i] * shape[i] && t.back() == ds[i] * shape[i]) {
            sh.back() *= shape[i], s.back() = ss[i], t.back() = ds[i];
        } else {
            sh.push_back(shape[i]), s.push_back(ss[i]), t.push_back(ds[i]);
        }
    }
    if (sh.empty())
        sh = {1}, s = {1}, t = {1};
    if (sh.size() > 6)
        return ESPDL_ERR_UNSUPPORTED;
    espdl_copy_desc d;
    memset(&d, 0, sizeof(d));
    d.src = src, d.dst = dst, d.elem_size = es, d.ndim = (int)sh.size();
    for (size_t i = 0; i < sh.size(); i++) d.shape[i] = sh[i], d.src_stride[i] = s[i], d.dst_stride[i] = t[i];
    return espdl_b200_copy(&d, ctx->stream);
}

static std::vector<long long> dense_strides(const std::vector<int> &shape)
{
    std::vector<long long> st(shape.size(), 1);
    for (int i = (int)shape.size() - 2; i >= 0; i--) st[i] = st[i + 1] * shape[i + 1];
    return st;
}

// Element strides of a tensor's device copy: dense, or with the rows of the last axis `row_stride` apart (a channel slice).
static std::vector<long long> device_strides(const TensorBase *t)
{
    std::vector<long long> st = dense_strides(t->shape);
    if (t->row_stride && t->shape.size() >= 2) {
        const int nd = (int)t->shape.size();
        st[nd - 2] = t->row_stride;
        for (int i = nd - 3; i >= 0; i--) st[i] = st[i + 1] * t->shape[i + 1];
    }
    return st;
}

std::vector<std::vector<int>> Concat::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    const int nd = (int)input_shapes[0].size();
    if (axis < 0)
        axis += nd;
    std::vector<int> out = input_shapes[0];
    out[axis] = 0;
    for (auto &s : input_shapes) out[axis] += s[axis];
    return {out};
}

// Concat / Split as one launch when every part is whole, aligned 16-byte units per row (rows = the extents before the axis);
// returns false when the shapes call for the strided copies instead.
static bool parts_in_one_launch(ModelContext *context, TensorBase *wide, const std::vector<TensorBase *> &parts, int axis, bool split, int &st)
{
    if (parts.empty() || parts.size() > 8 || !wide || !wide->device || ((uintptr_t)wide->device % 16))
        return false;
    const long long es = (long long)dtype_sizeof(wide->dtype);
    long long rows = 1, inner = es;
    for (int i = 0; i < axis; i++) rows *= wide->shape[i];
    for (size_t i = axis + 1; i < wide->shape.size(); i++) inner *= wide->shape[i];
    espdl_parts_desc d;
    memset(&d, 0, sizeof(d));
    d.wide = wide->device, d.n_parts = (int)parts.size(), d.split = split ? 1 : 0, d.rows = rows;
    long long at = 0, wide_row = 0;
    for (TensorBase *t : parts)
        if (t && (int)t->shape.size() == (int)wide->shape.size())
            wide_row += (long long)t->shape[axis] * inner;
    int to_move = 0;
    for (size_t i = 0; i < parts.size(); i++) {
        TensorBase *t = parts[i];
        if (!t || !t->device || ((uintptr_t)t->device % 16) || t->dtype != wide->dtype || (int)t->shape.size() != (int)wide->shape.size())
            return false;
        d.parts[i] = t->device;
        d.part_bytes[i] = (long long)t->shape[axis] * inner;
        if (d.part_bytes[i] % 16 != 0)
            return false;
        if (t->row_stride) { // a channel slice: already inside the wide tensor (nothing to move), or rows apart elsewhere
            d.part_stride[i] = (long long)t->row_stride * es;
            if ((char *)t->device == (char *)wide->device + at && d.part_stride[i] == wide_row)
                d.skip[i] = 1;
        }
        to_move += d.skip[i] ? 0 : 1;
        at += d.part_bytes[i];
    }
    st = to_move ? espdl_b200_concat_split(&d, context->stream) : ESPDL_OK;
    return true;
}

// Last axis, at most eight parts, every part whole 16-byte units per row: the one-launch form, which also moves slices.
static bool parts_are_units(const std::vector<std::vector<int>> &shapes, int axis, int es)
{
    if (shapes.empty() || shapes.size() > 8 || shapes[0].size() < 2)
        return false;
    const int nd = (int)shapes[0].size();
    if ((axis < 0 ? axis + nd : axis) != nd - 1)
        return false;
    for (const std::vector<int> &s : shapes)
        if ((int)s.size() != nd || ((long long)s.back() * es) % 16 != 0)
            return false;
    return true;
}

static int quant_elem_size(quant_type_t q) { return q == QUANT_TYPE_SYMM_16BIT ? 2 : 1; }

bool Concat::strided_input_ok(int i, const std::vector<std::vector<int>> &in) const
{
    return i >= 0 && i < (int)in.size() && quant_type != QUANT_TYPE_NONE && parts_are_units(in, axis, quant_elem_size(quant_type));
}

bool Split::strided_output_ok(int o, const std::vector<std::vector<int>> &in) const
{
    if (o < 0 || in.empty() || quant_type == QUANT_TYPE_NONE)
        return false;
    std::vector<std::vector<int>> shapes = in;
    shapes.resize(1);
    std::vector<std::vector<int>> outs = const_cast<Split *>(this)->get_output_shape(shapes);
    return o < (int)outs.size() && parts_are_units(outs, m_axis, quant_elem_size(quant_type));
}

void Concat::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    const int es = (int)dtype_sizeof(out->dtype);
    const std::vector<long long> os = dense_strides(out->shape);
    long long offset = 0;
    int st = ESPDL_OK;
    {
        std::vector<TensorBase *> parts;
        for (int idx : m_inputs_index) parts.push_back(context->get_tensor(idx));
        const int ax = axis < 0 ? axis + (int)out->shape.size() : axis;
        if (parts_in_one_launch(context, out, parts, ax, false, st)) {
            if (st)
                ESP_LOGE("Concat", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
            context->note(st);
            return;
        }
    }
    for (size_t i = 0; i < m_inputs_index.size() && !st; i++) {
        TensorBase *in = context->get_tensor(m_inputs_index[i]);
        if (!in || !in->device || !out->device) {
            st = ESPDL_ERR_INVALID_ARG;
            break;
        }
        char *place = (char *)out->device + offset * os[axis] * es;
        offset += in->shape[axis];
        if (in->row_stride && (char *)in->device == place && in->row_stride == out->shape.back())
            continue; // a slice of this very output: its producer wrote it in place
        st = enqueue_copy(context, in->device, place, es, in->shape, device_strides(in), os);
    }
    if (st)
        ESP_LOGE("Concat", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

Module *Concat::deserialize(fbs::FbsModel *m, std::string node)
{
    int axis = 0;
    m->get_operation_attribute(node, "axis", axis);
    return new Concat(node.c_str(), axis, node_quant(m, node));
}

Split::Split(TensorBase *split, int axis, int num_outputs, const char *name, module_inplace_t inplace, quant_type_t quant_type) :
    Module(name, inplace, quant_type), m_axis(axis), m_num_outputs(num_outputs)
{
    if (split && split->data) {
        for (int i = 0; i < split->get_size(); i++)
            m_split.push_back(split->dtype == DATA_TYPE_INT64 ? (int)((int64_t *)split->data)[i] : ((int32_t *)split->data)[i]);
    }
    delete split;
}

std::vector<std::vector<int>> Split::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    std::vector<int> in = input_shapes[0];
    if (m_axis < 0)
        m_axis += (int)in.size();
    if (m_split.empty()) {
        const int n = m_num_outputs > 0 ? m_num_outputs : 2;
        const int each = (in[m_axis] + n - 1) / n;
        for (int i = 0; i < n; i++) m_split.push_back(std::min(each, in[m_axis] - i * each));
    }
    std::vector<std::vector<int>> outs;
    for (int s : m_split) {
        std::vector<int> o = in;
        o[m_axis] = s;
        outs.push_back(o);
    }
    return outs;
}

void Split::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *in = context->get_tensor(m_inputs_index[0]);
    const int es = (int)dtype_sizeof(in->dtype);
    const std::vector<long long> is = dense_strides(in->shape);
    long long offset = 0;
    int st = ESPDL_OK;
    {
        std::vector<TensorBase *> parts;
        for (int idx : m_outputs_index) parts.push_back(context->get_tensor(idx));
        if (parts_in_one_launch(context, in, parts, m_axis, true, st)) {
            if (st)
                ESP_LOGE("Split", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
            context->note(st);
            return;
        }
    }
    for (size_t i = 0; i < m_outputs_index.size() && !st; i++) {
        TensorBase *out = context->get_tensor(m_outputs_index[i]);
        if (!out || !out->device || !in->device) {
            st = ESPDL_ERR_INVALID_ARG;
            break;
        }
        char *place = (char *)in->device + offset * is[m_axis] * es;
        offset += out->shape[m_axis];
        if (out->row_stride && (char *)out->device == place && out->row_stride == in->shape.back())
            continue; // a window into this very input
        st = enqueue_copy(context, place, out->device, es, out->shape, is, device_strides(out));
    }
    if (st)
        ESP_LOGE("Split", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

Module *Split::deserialize(fbs::FbsModel *m, std::string node)
{
    int axis = 0, num_outputs = -1;
    m->get_operation_attribute(node, "axis", axis);
    m->get_operation_attribute(node, "num_outputs", num_outputs);
    return new Split(m->get_operation_parameter(node, 1), axis, num_outputs, node.c_str(), MODULE_NON_INPLACE, node_quant(m, node));
}

// --------------------------------------------------------------------------------- Reduce / Slice
std::vector<std::vector<int>> Reduce::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    // dl_module_reduce_base.hpp:43-70
    const std::vector<int> &in = input_shapes[0];
    std::vector<int> out;
    size_t reduced = 0;
    for (size_t i = 0; i < in.size(); i++) {
        if (i < m_axes_reduce_flag.size() && m_axes_reduce_flag[i]) {
            reduced++;
            if (m_keepdims)
                out.push_back(1);
        } else {
            out.push_back(in[i]);
        }
    }
    if (!m_keepdims && reduced == in.size())
        out = {1};
    return {out};
}

// tool::gen_lut_8bit(expf) (esp-dl/dl/tool/src/dl_tool.cpp:258-268) on the device; rebuilt when the exponent changes
static int upload_exp_table(void *&dev, int &have_exponent, int exponent)
{
    if (dev && have_exponent == exponent)
        return ESPDL_OK;
    float table[256];
    const float scale = DL_SCALE(exponent);
    for (int i = 0; i < 256; i++) table[i] = expf(scale * (float)(i - 128));
    if (!dev && espdl_b200_arena_alloc(sizeof(table), &dev) != ESPDL_OK)
        return ESPDL_ERR_NO_MEM;
    int st = espdl_b200_upload(dev, table, sizeof(table), nullptr);
    if (!st)
        st = espdl_b200_stream_sync(nullptr);
    have_exponent = exponent;
    return st;
}

Reduce::~Reduce()
{
    if (m_dev_table)
        espdl_b200_arena_free(m_dev_table);
}

void Reduce::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *in = context->get_tensor(m_inputs_index[0]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    int st = ESPDL_OK;
    espdl_reduce_desc d;
    memset(&d, 0, sizeof(d));
    if (!in || !out || !in->device || !out->device || in->shape.size() > 6 || in->shape.empty()) {
        st = ESPDL_ERR_INVALID_ARG;
    } else if (m_op == ESPDL_REDUCE_LOG_SUM_EXP && quant_type != QUANT_TYPE_SYMM_16BIT &&
               (st = upload_exp_table(m_dev_table, m_table_exponent, (int)in->exponent)) != ESPDL_OK) {
    } else {
        d.exp_table = (const float *)m_dev_table;
        d.input = in->device, d.output = out->device, d.op = m_op, d.dtype = quant_dtype(quant_type), d.ndim = (int)in->shape.size();
        for (size_t i = 0; i < in->shape.size(); i++) d.shape[i] = in->shape[i], d.reduce[i] = i < m_axes_reduce_flag.size() && m_axes_reduce_flag[i];
        d.in_exponent = in->exponent, d.out_exponent = out->exponent, d.round_mode = context->round_mode;
        st = espdl_b200_reduce(&d, context->stream);
    }
    if (st)
        ESP_LOGE("Reduce", "%s failed: %s %s", name ? name : "?", espdl_b200_strerror(st), espdl_b200_last_error());
    context->note(st);
}

Module *Reduce::deserialize(fbs::FbsModel *m, std::string node)
{
    // ReduceBase::get_attributes, dl_module_reduce_base.hpp:265-298
    const std::string type = m->get_operation_type(node);
    int op = ESPDL_REDUCE_MIN;
    for (auto &kv : std::initializer_list<std::pair<const char *, int>>{{"ReduceMean", ESPDL_REDUCE_MEAN}, {"ReduceSum", ESPDL_REDUCE_SUM},
                                                                       {"ReduceMax", ESPDL_REDUCE_MAX}, {"ReduceL1", ESPDL_REDUCE_L1},
                                                                       {"ReduceSumSquare", ESPDL_REDUCE_SUM_SQUARE}, {"ReduceL2", ESPDL_REDUCE_L2},
                                                                       {"ReduceProd", ESPDL_REDUCE_PROD}, {"ReduceLogSum", ESPDL_REDUCE_LOG_SUM},
                                                                       {"ReduceLogSumExp", ESPDL_REDUCE_LOG_SUM_EXP}})
        if (type == kv.first)
            op = kv.second;
    int keepdims = 1, noop = 0;
    m->get_operation_attribute(node, "keepdims", keepdims);
    m->get_operation_attribute(node, "noop_with_empty_axes", noop);
    std::vector<std::string> ins, outs;
    m->get_operation_inputs_and_outputs(node, ins, outs);
    const std::vector<int> in_shape = ins.empty() ? std::vector<int>() : m->get_value_info_shape(ins[0]);
    std::vector<bool> flags(in_shape.size(), false);
    TensorBase *axes = m->get_operation_parameter(node, 1);
    if (axes && axes->get_size() > 0) {
        for (int i = 0; i < axes->get_size(); i++) {
            int a = axes->dtype == DATA_TYPE_INT64 ? (int)axes->get_element<int64_t>(i) : axes->get_element<int32_t>(i);
            if (a < 0)
                a += (int)in_shape.size();
            if (a >= 0 && a < (int)flags.size())
                flags[a] = true;
        }
    } else if (!noop) {
        std::fill(flags.begin(), flags.end(), true);
    }
    delete axes;
    const quant_type_t q = node_quant(m, node);
    if (q != QUANT_TYPE_SYMM_8BIT && q != QUANT_TYPE_SYMM_16BIT)
        return nullptr;
    return new Reduce(op, keepdims, flags, node.c_str(), q);
}

bool Slice::resolve(const std::vector<int> &shape, std::vector<int> &first, std::vector<int> &count, std::vector<int> &step) const
{
    // get_slice_shape / _slice: dl_base_shape.cpp:68-120, dl_tensor_base.cpp:1049-1100 (positive steps)
    const int dims = (int)shape.size();
    first.assign(dims, 0), step.assign(dims, 1);
    count = shape;
    for (size_t i = 0; i < m_start.size(); i++) {
        int axis = (int)i;
        if (!m_axes.empty())
            axis = (m_axes[i] + dims) % dims;
        const int st = m_step.empty() ? 1 : m_step[i];
        if (st <= 0 || axis < 0 || axis >= dims)
            return false;
        int s0 = m_start[i], e0 = m_end[i];
        if (e0 > shape[axis])
            e0 = shape[axis];
        else if (e0 < 0)
            e0 += shape[axis];
        if (s0 > shape[axis])
            s0 = shape[axis];
        else if (s0 < 0)
            s0 += shape[axis];
        if (s0 < 0 || s0 >= e0)
            return false;
        first[axis] = s0, step[axis] = st, count[axis] = 1 + (e0 - s0 - 1) / st;
    }
    return true;
}

std::vector<std::vector<int>> Slice::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    std::vector<int> first, count, step;
    if (!resolve(input_shapes[0], first, count, step))
        return {{}};
    return {count};
}

void Slice::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *in = context->get_tensor(m_inputs_index[0]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    int st = ESPDL_OK;
    std::vector<int> first, count, step;
    if (!in || !out || !in->device || !out->device || !resolve(in->shape, first, count, step)) {
        st = ESPDL_ERR_INVALID_ARG;
    } else {
        const int es = (int)dtype_sizeof(in->dtype);
        std::vector<long long> is = dense_strides(in->shape);
        long long offset = 0;
        for (size_t i = 0; i < is.size(); i++) {
            offset += (long long)first[i] * is[i];
            is[i] *= step[i];
        }
        st = enqueue_copy(context, (char *)in->device + offset * es, out->device, es, count, is, dense_strides(count));
    }
    if (st)
        ESP_LOGE("Slice", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

Module *Slice::deserialize(fbs::FbsModel *m, std::string node)
{
    // dl_module_slice.hpp:58-121; negative steps (the reference flips those axes) are not taken
    TensorBase *p[4] = {m->get_operation_parameter(node, 1), m->get_operation_parameter(node, 2), m->get_operation_parameter(node, 3),
                        m->get_operation_parameter(node, 4)};
    std::vector<int> v[4];
    bool ok = p[0] && p[1];
    for (int k = 0; k < 4 && ok; k++) {
        if (!p[k])
            continue;
        for (int i = 0; i < p[k]->get_size(); i++) {
            long long x = p[k]->dtype == DATA_TYPE_INT64 ? (long long)p[k]->get_element<int64_t>(i) : (long long)p[k]->get_element<int32_t>(i);
            x = x > INT32_MAX ? INT32_MAX : (x < INT32_MIN ? INT32_MIN : x); // tool::truncate
            v[k].push_back((int)x);
        }
    }
    for (int k = 0; k < 4; k++) delete p[k];
    for (int s : v[3])
        if (s <= 0)
            ok = false;
    if (!ok) {
        ESP_LOGE("Slice", "%s: missing bounds or a step that is not positive", node.c_str());
        return nullptr;
    }
    return new Slice(v[0], v[1], v[2], v[3], node.c_str(), node_quant(m, node));
}

std::vector<std::vector<int>> Pad::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    std::vector<int> out = input_shapes[0];
    const size_t n = out.size();
    for (size_t i = 0; i < n && n + i < m_pads.size(); i++) out[i] += m_pads[i] + m_pads[n + i];
    return {out};
}

void Pad::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *in = context->get_tensor(m_inputs_index[0]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    int st = ESPDL_OK;
    espdl_pad_desc d;
    memset(&d, 0, sizeof(d));
    const size_t n = in ? in->shape.size() : 0;
    if (!in || !out || !in->device || !out->device || n == 0 || n > 6 || m_pads.size() != 2 * n) {
        st = ESPDL_ERR_INVALID_ARG;
    } else {
        d.input = in->device, d.output = out->device, d.elem_size = (int)dtype_sizeof(in->dtype), d.ndim = (int)n, d.mode = m_mode;
        for (size_t i = 0; i < n; i++) d.shape[i] = in->shape[i], d.pad_begin[i] = m_pads[i], d.pad_end[i] = m_pads[n + i];
        d.constant = m_constant;
        st = espdl_b200_pad(&d, context->stream);
    }
    if (st)
        ESP_LOGE("Pad", "%s failed: %s %s", name ? name : "?", espdl_b200_strerror(st), espdl_b200_last_error());
    context->note(st);
}

Module *Pad::deserialize(fbs::FbsModel *m, std::string node)
{
    std::string mode = "constant";
    m->get_operation_attribute(node, "mode", mode);
    const int pm = mode == "constant" ? ESPDL_PAD_CONSTANT : (mode == "edge" ? ESPDL_PAD_EDGE : (mode == "reflect" ? ESPDL_PAD_REFLECT : -1));
    TensorBase *pads = m->get_operation_parameter(node, 1);
    TensorBase *cv = m->get_operation_parameter(node, 2);
    if (pm < 0 || !pads || pads->dtype != DATA_TYPE_INT64) {
        ESP_LOGE("Pad", "%s: mode %s or pads are not supported", node.c_str(), mode.c_str());
        delete pads;
        delete cv;
        return nullptr;
    }
    std::vector<int> p;
    for (int i = 0; i < pads->get_size(); i++) p.push_back((int)pads->get_element<int64_t>(i));
    long long c = 0;
    if (cv && cv->get_size() > 0)
        c = cv->dtype == DATA_TYPE_INT8 ? cv->get_element<int8_t>(0) : (cv->dtype == DATA_TYPE_INT16 ? cv->get_element<int16_t>(0) : 0);
    delete pads;
    delete cv;
    return new Pad(p, pm, c, node.c_str(), node_quant(m, node));
}

std::vector<std::vector<int>> Transpose::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    std::vector<int> in = input_shapes[0], out(in.size());
    if (m_perm.empty())
        for (int i = (int)in.size() - 1; i >= 0; i--) m_perm.push_back(i);
    if (m_perm.size() != in.size()) {
        ESP_LOGE("Transpose", "%s: perm has %d entries for a tensor of rank %d", name ? name : "?", (int)m_perm.size(), (int)in.size());
        return {{}};
    }
    for (size_t i = 0; i < in.size(); i++) {
        if (m_perm[i] < 0) // negative entries count from the last axis (dl_module_transpose.hpp:43-46)
            m_perm[i] += (int)m_perm.size();
        if (m_perm[i] < 0 || m_perm[i] >= (int)in.size())
            return {{}};
        out[i] = in[m_perm[i]];
    }
    return {out};
}

void Transpose::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *in = context->get_tensor(m_inputs_index[0]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    int st = (!in || !out || !in->device || !out->device) ? ESPDL_ERR_INVALID_ARG : ESPDL_OK;
    if (!st) {
        const std::vector<long long> is = dense_strides(in->shape);
        std::vector<long long> ss(out->shape.size());
        for (size_t i = 0; i < out->shape.size(); i++) ss[i] = is[m_perm[i]];
        st = enqueue_copy(context, in->device, out->device, (int)dtype_sizeof(in->dtype), out->shape, ss, dense_strides(out->shape));
    }
    if (st)
        ESP_LOGE("Transpose", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

Module *Transpose::deserialize(fbs::FbsModel *m, std::string node)
{
    std::vector<int> perm;
    m->get_operation_attribute(node, "perm", perm);
    return new Transpose(node.c_str(), MODULE_NON_INPLACE, node_quant(m, node), perm);
}

// --------------------------------------------------------------------------------- SpaceToDepth / DepthToSpace / Gather
std::vector<std::vector<int>> SpaceToDepth::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    std::vector<int> in = input_shapes[0], out = in;
    if (in.size() != 4 || m_blocksize < 1 || in[1] % m_blocksize || in[2] % m_blocksize) {
        ESP_LOGE("SpaceToDepth", "input must be [N, H, W, C] with H and W divisible by blocksize %d", m_blocksize);
        return {in};
    }
    out[1] = in[1] / m_blocksize, out[2] = in[2] / m_blocksize, out[3] = in[3] * m_blocksize * m_blocksize;
    return {out};
}

void SpaceToDepth::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *in = context->get_tensor(m_inputs_index[0]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    int st = (!in || !out || !in->device || !out->device || in->shape.size() != 4 || out->shape.size() != 4) ? ESPDL_ERR_INVALID_ARG : ESPDL_OK;
    if (!st && (in->shape[1] % m_blocksize || in->shape[2] % m_blocksize || in->get_size() != out->get_size()))
        st = ESPDL_ERR_INVALID_ARG;
    if (!st) {
        // out[n][oh][ow][c][hb][wb] = in[n][oh*bs + hb][ow*bs + wb][c]  (dl_module_space_to_depth.hpp:31-40)
        const long long bs = m_blocksize, W = in->shape[2], Cc = in->shape[3], H = in->shape[1];
        const std::vector<int> shape = {in->shape[0], (int)(H / bs), (int)(W / bs), (int)Cc, (int)bs, (int)bs};
        const std::vector<long long> ss = {H * W * Cc, bs * W * Cc, bs * Cc, 1, W * Cc, Cc};
        st = enqueue_copy(context, in->device, out->device, (int)dtype_sizeof(in->dtype), shape, ss, dense_strides(shape));
    }
    if (st)
        ESP_LOGE("SpaceToDepth", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

Module *SpaceToDepth::deserialize(fbs::FbsModel *m, std::string node)
{
    int blocksize = 2;
    m->get_operation_attribute(node, "blocksize", blocksize);
    return new SpaceToDepth(blocksize, node.c_str(), MODULE_NON_INPLACE, node_quant(m, node));
}

std::vector<std::vector<int>> DepthToSpace::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    std::vector<int> in = input_shapes[0], out = in;
    if (in.size() != 4 || m_blocksize < 1 || in[3] % (m_blocksize * m_blocksize)) {
        ESP_LOGE("DepthToSpace", "input must be [N, H, W, C] with C divisible by blocksize^2");
        return {in};
    }
    out[1] = in[1] * m_blocksize, out[2] = in[2] * m_blocksize, out[3] = in[3] / (m_blocksize * m_blocksize);
    return {out};
}

void DepthToSpace::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *in = context->get_tensor(m_inputs_index[0]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    int st = (!in || !out || !in->device || !out->device || in->shape.size() != 4 || out->shape.size() != 4) ? ESPDL_ERR_INVALID_ARG : ESPDL_OK;
    const long long bs = m_blocksize;
    if (!st && (in->shape[3] % (bs * bs) || in->get_size() != out->get_size()))
        st = ESPDL_ERR_INVALID_ARG;
    const bool crd = m_mode == "CRD";
    if (!st && !crd && in->shape[3] / (bs * bs) != bs) // see the class comment
        st = ESPDL_ERR_UNSUPPORTED;
    if (!st) {
        // out[n][h][hb][w][wb][co] = in[n][h][w][c], c = co*bs*bs + hb*bs + wb (CRD) or hb*bs*bs + wb*bs + co (DCR, co < bs)
        const long long H = in->shape[1], W = in->shape[2], Cc = in->shape[3], Co = Cc / (bs * bs);
        const std::vector<int> shape = {in->shape[0], (int)H, (int)bs, (int)W, (int)bs, (int)Co};
        const std::vector<long long> ss = crd ? std::vector<long long>{H * W * Cc, W * Cc, bs, Cc, 1, bs * bs}
                                              : std::vector<long long>{H * W * Cc, W * Cc, bs * bs, Cc, bs, 1};
        st = enqueue_copy(context, in->device, out->device, (int)dtype_sizeof(in->dtype), shape, ss, dense_strides(shape));
    }
    if (st)
        ESP_LOGE("DepthToSpace", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

Module *DepthToSpace::deserialize(fbs::FbsModel *m, std::string node)
{
    int blocksize = 2;
    std::string mode;
    m->get_operation_attribute(node, "blocksize", blocksize);
    m->get_operation_attribute(node, "mode", mode);
    return new DepthToSpace(blocksize, mode.empty() ? "DCR" : mode, node.c_str(), MODULE_NON_INPLACE, node_quant(m, node));
}

std::vector<std::vector<int>> InsertZeros::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    // dl_module_insert_zeros.hpp:33-58
    std::vector<int> in = input_shapes[0], out = in;
    if (in.size() != 3 && in.size() != 4) {
        ESP_LOGE("InsertZeros", "%s: one or two spatial axes expected", name ? name : "?");
        return {{}};
    }
    const int spatial = (int)in.size() - 2;
    if (m_stride.size() == 1 && spatial > 1)
        m_stride.assign(spatial, m_stride[0]);
    if (m_output_padding.size() == 1 && spatial > 1)
        m_output_padding.assign(spatial, m_output_padding[0]);
    if ((int)m_stride.size() != spatial || (int)m_output_padding.size() != spatial)
        return {{}};
    for (int i = 0; i < spatial; i++) out[1 + i] = in[1 + i] + (m_stride[i] - 1) * (in[1 + i] - 1) + m_output_padding[i];
    return {out};
}

void InsertZeros::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *in = context->get_tensor(m_inputs_index[0]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    int st = (!in || !out || !in->device || !out->device || in->shape.size() != out->shape.size() ||
              in->shape.size() != m_stride.size() + 2) ? ESPDL_ERR_INVALID_ARG : ESPDL_OK;
    if (!st)
        st = espdl_b200_memset(out->device, 0, (size_t)out->get_size() * dtype_sizeof(out->dtype), context->stream);
    if (!st) {
        std::vector<long long> ds = dense_strides(out->shape);
        for (size_t i = 0; i < m_stride.size(); i++) ds[1 + i] *= m_stride[i];
        st = enqueue_copy(context, in->device, out->device, (int)dtype_sizeof(in->dtype), in->shape, dense_strides(in->shape), ds);
    }
    if (st)
        ESP_LOGE("InsertZeros", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

Module *InsertZeros::deserialize(fbs::FbsModel *m, std::string node)
{
    std::vector<int> stride, output_padding;
    m->get_operation_attribute(node, "stride", stride);
    m->get_operation_attribute(node, "output_padding", output_padding);
    if (stride.empty())
        stride = {1};
    if (output_padding.empty())
        output_padding = {0};
    for (int v : stride)
        if (v < 1)
            return nullptr;
    return new InsertZeros(node.c_str(), stride, output_padding, node_quant(m, node));
}

StreamingCache::~StreamingCache()
{
    if (m_cache)
        espdl_b200_arena_free(m_cache);
}

std::vector<std::vector<int>> StreamingCache::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    std::vector<int> out = input_shapes[0];
    if (m_frame_axis < 0)
        m_frame_axis += (int)out.size();
    if (m_frame_axis < 0 || m_frame_axis >= (int)out.size() || m_window_size < 1) {
        ESP_LOGE("StreamingCache", "%s: frame_axis outside the tensor", name ? name : "?");
        return {{}};
    }
    out[m_frame_axis] += m_window_size - 1;
    return {out};
}

esp_err_t StreamingCache::prepare(ModelContext *context)
{
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    if (!out || m_frame_axis < 0 || m_frame_axis >= (int)out->shape.size())
        return ESP_FAIL;
    size_t n = dtype_sizeof(out->dtype) * (size_t)(m_window_size - 1);
    for (int i = 0; i < (int)out->shape.size(); i++)
        if (i != m_frame_axis)
            n *= (size_t)out->shape[i];
    if (m_cache)
        espdl_b200_arena_free(m_cache);
    m_cache = nullptr, m_cache_bytes = n;
    if (n == 0)
        return ESP_OK;
    if (espdl_b200_arena_alloc(n, &m_cache) != ESPDL_OK || espdl_b200_memset(m_cache, 0, n, nullptr) != ESPDL_OK ||
        espdl_b200_stream_sync(nullptr) != ESPDL_OK)
        return ESP_FAIL;
    return ESP_OK;
}

void StreamingCache::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *in = context->get_tensor(m_inputs_index[0]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    int st = (!in || !out || !in->device || !out->device) ? ESPDL_ERR_INVALID_ARG : ESPDL_OK;
    const size_t in_bytes = in ? (size_t)in->get_size() * dtype_sizeof(in->dtype) : 0;
    if (!st && (size_t)out->get_size() * dtype_sizeof(out->dtype) != in_bytes + m_cache_bytes)
        st = ESPDL_ERR_INVALID_ARG;
    auto copy_bytes = [&](const void *src, void *dst, size_t n) {
        return n ? enqueue_copy(context, src, dst, 1, {(int)n}, {1}, {1}) : ESPDL_OK;
    };
    // dl_module_streaming_cache.hpp:56-70
    if (!st && m_cache_bytes)
        st = copy_bytes(m_cache, out->device, m_cache_bytes);
    if (!st)
        st = copy_bytes(in->device, (char *)out->device + m_cache_bytes, in_bytes);
    if (!st && m_cache_bytes)
        st = copy_bytes((char *)out->device + in_bytes, m_cache, m_cache_bytes);
    if (st)
        ESP_LOGE("StreamingCache", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

void StreamingCache::reset()
{
    if (m_cache && m_cache_bytes) {
        espdl_b200_memset(m_cache, 0, m_cache_bytes, nullptr);
        espdl_b200_stream_sync(nullptr);
    }
}

Module *StreamingCache::deserialize(fbs::FbsModel *m, std::string node)
{
    int window_size = 1, frame_axis = 1;
    m->get_operation_attribute(node, "window_size", window_size);
    m->get_operation_attribute(node, "frame_axis", frame_axis);
    return new StreamingCache(node.c_str(), window_size, frame_axis, MODULE_NON_INPLACE, node_quant(m, node));
}

Gather::~Gather()
{
    delete m_indices;
    delete m_dev_indices;
}

std::vector<std::vector<int>> Gather::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    const std::vector<int> &in = input_shapes[0];
    if (m_axis < 0)
        m_axis += (int)in.size();
    std::vector<int> out;
    for (int i = 0; i < (int)in.size(); i++) {
        if (i == m_axis && m_indices)
            out.insert(out.end(), m_indices->shape.begin(), m_indices->shape.end());
        else
            out.push_back(in[i]);
    }
    return {out};
}

esp_err_t Gather::prepare(ModelContext *context)
{
    TensorBase *in = context->get_tensor(m_inputs_index[0]);
    if (!in || !m_indices || m_axis < 0 || m_axis >= (int)in->shape.size())
        return ESP_FAIL;
    if (m_indices->dtype != DATA_TYPE_INT64 && m_indices->dtype != DATA_TYPE_INT32)
        return ESP_FAIL;
    std::vector<int32_t> idx(m_indices->get_size());
    for (int i = 0; i < m_indices->get_size(); i++) {
        const long long v = m_indices->dtype == DATA_TYPE_INT64 ? (long long)m_indices->get_element<int64_t>(i) : m_indices->get_element<int32_t>(i);
        if (v < 0 || v >= in->shape[m_axis]) { // the reference would read outside the tensor
            ESP_LOGE("Gather", "%s: index %lld outside [0, %d)", name ? name : "?", v, in->shape[m_axis]);
            return ESP_FAIL;
        }
        idx[i] = (int32_t)v;
    }
    delete m_dev_indices;
    m_dev_indices = new TensorBase({(int)idx.size()}, idx.data(), 0, DATA_TYPE_INT32, true);
    if (m_dev_indices->to_device() != ESP_OK || espdl_b200_stream_sync(nullptr) != ESPDL_OK)
        return ESP_FAIL;
    return ESP_OK;
}

void Gather::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *in = context->get_tensor(m_inputs_index[0]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    int st = (!in || !out || !in->device || !out->device || !m_dev_indices || !m_dev_indices->device) ? ESPDL_ERR_INVALID_ARG : ESPDL_OK;
    if (!st) {
        espdl_gather_desc d;
        memset(&d, 0, sizeof(d));
        d.input = in->device, d.output = out->device, d.indices = (const int32_t *)m_dev_indices->device;
        d.elem_size = (int)dtype_sizeof(in->dtype), d.num_indices = m_dev_indices->get_size();
        d.outer = 1, d.inner = 1, d.axis_size = in->shape[m_axis];
        for (int i = 0; i < m_axis; i++) d.outer *= in->shape[i];
        for (size_t i = m_axis + 1; i < in->shape.size(); i++) d.inner *= in->shape[i];
        st = espdl_b200_gather(&d, context->stream);
    }
    if (st)
        ESP_LOGE("Gather", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

Module *Gather::deserialize(fbs::FbsModel *m, std::string node)
{
    int axis = 0;
    m->get_operation_attribute(node, "axis", axis);
    TensorBase *indices = m->get_operation_parameter(node, 1);
    if (!indices)
        return nullptr;
    return new Gather(indices, axis, node.c_str(), MODULE_NON_INPLACE, node_quant(m, node));
}

// --------------------------------------------------------------------------------- RMSNormalization / LayerNormalization
std::vector<std::vector<int>> Normalization::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    const std::vector<int> &x = input_shapes[0];
    if (m_op == ESPDL_NORM_RMS)
        return {x};
    // LayerNormalization::calculate_normalized_shape, dl_module_layer_normalization.hpp:186-196
    const int axis = m_axis < 0 ? (int)x.size() + m_axis : m_axis;
    std::vector<int> stat(x.size(), 1);
    for (int i = 0; i < axis && i < (int)x.size(); i++) stat[i] = x[i];
    return {x, stat, stat};
}

esp_err_t Normalization::prepare(ModelContext *context)
{
    for (size_t i = 1; i < m_inputs_index.size(); i++) {
        TensorBase *t = context->get_tensor(m_inputs_index[i]);
        if (t && t->data && !t->device && t->to_device() != ESP_OK)
            return ESP_FAIL;
    }
    return espdl_b200_stream_sync(nullptr) == ESPDL_OK ? ESP_OK : ESP_FAIL;
}

void Normalization::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *x = context->get_tensor(m_inputs_index[0]);
    TensorBase *scale = m_inputs_index.size() > 1 ? context->get_tensor(m_inputs_index[1]) : nullptr;
    TensorBase *bias = m_inputs_index.size() > 2 ? context->get_tensor(m_inputs_index[2]) : nullptr;
    TensorBase *y = context->get_tensor(m_outputs_index[0]);
    TensorBase *mean = m_outputs_index.size() > 1 ? context->get_tensor(m_outputs_index[1]) : nullptr;
    TensorBase *inv = m_outputs_index.size() > 2 ? context->get_tensor(m_outputs_index[2]) : nullptr;
    espdl_norm_desc d;
    memset(&d, 0, sizeof(d));
    int st = (!x || !y || !x->device || !y->device) ? ESPDL_ERR_INVALID_ARG : ESPDL_OK;
    if (!st && m_op == ESPDL_NORM_RMS && (!scale || !scale->device || scale->dtype != DATA_TYPE_FLOAT))
        st = ESPDL_ERR_INVALID_ARG;
    if (!st && ((scale && !scale->device) || (bias && !bias->device) || (mean && !mean->device) || (inv && !inv->device)))
        st = ESPDL_ERR_INVALID_ARG;
    if (!st) {
        const int axis = m_axis < 0 ? (int)x->shape.size() + m_axis : m_axis;
        long long rows = 1, len = 1;
        for (int i = 0; i < (int)x->shape.size(); i++) (i < axis ? rows : len) *= x->shape[i];
        d.input = x->device, d.output = y->device, d.op = m_op, d.dtype = quant_dtype(quant_type);
        d.scale = scale ? scale->device : nullptr, d.bias = bias ? bias->device : nullptr;
        d.mean = mean ? mean->device : nullptr, d.inv_std_dev = inv ? inv->device : nullptr;
        d.rows = rows, d.len = (int)len;
        d.in_exponent = x->exponent, d.out_exponent = y->exponent;
        d.scale_exponent = scale ? (int)scale->exponent : 0, d.bias_exponent = bias ? (int)bias->exponent : 0;
        d.mean_exponent = mean ? (int)mean->exponent : 0, d.inv_std_dev_exponent = inv ? (int)inv->exponent : 0;
        d.epsilon = m_epsilon, d.round_mode = context->round_mode;
        if (len > INT_MAX || (scale && scale->get_size() < len) || (bias && bias->get_size() < len))
            st = ESPDL_ERR_INVALID_ARG;
        else
            st = espdl_b200_norm(&d, context->stream);
    }
    if (st)
        ESP_LOGE("Normalization", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

RMSNormalization::RMSNormalization(int axis, float epsilon, const char *name, module_inplace_t inplace, quant_type_t quant_type) :
    Normalization(ESPDL_NORM_RMS, axis, epsilon, name, inplace, quant_type)
{
}

LayerNormalization::LayerNormalization(int axis, float epsilon, int stash_type, const char *name, module_inplace_t inplace,
                                       quant_type_t quant_type) :
    Normalization(ESPDL_NORM_LAYER, axis, epsilon, name, inplace, quant_type)
{
    (void)stash_type;
}

static Module *deserialize_norm(fbs::FbsModel *m, const std::string &node, bool rms)
{
    int axis = -1;
    float epsilon = 1e-5f;
    m->get_operation_attribute(node, "axis", axis);
    m->get_operation_attribute(node, "epsilon", epsilon);
    const quant_type_t q = node_quant(m, node);
    if (q != QUANT_TYPE_SYMM_8BIT && q != QUANT_TYPE_SYMM_16BIT)
        return nullptr;
    if (rms)
        return new RMSNormalization(axis, epsilon, node.c_str(), MODULE_INPLACE_CHANGED_BUFFER, q);
    int stash_type = 1;
    m->get_operation_attribute(node, "stash_type", stash_type);
    return new LayerNormalization(axis, epsilon, stash_type, node.c_str(), MODULE_INPLACE_CHANGED_BUFFER, q);
}
Module *RMSNormalization::deserialize(fbs::FbsModel *m, std::string node) { return deserialize_norm(m, node, true); }
Module *LayerNormalization::deserialize(fbs::FbsModel *m, std::string node) { return deserialize_norm(m, node, false); }

std::vector<std::vector<int>> Reshape::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    std::vector<int> in = input_shapes[0], out;
    long long total = 1;
    for (int d : in) total *= d;
    switch (m_kind) {
    case RESHAPE: {
        out = m_arg;
        long long known = 1;
        int unknown = -1;
        for (size_t i = 0; i < out.size(); i++) {
            if (out[i] == 0 && i < in.size())
                out[i] = in[i];
            if (out[i] == -1)
                unknown = (int)i;
            else
                known *= out[i];
        }
        if (unknown >= 0)
            out[unknown] = (int)(total / known);
        else if (known != total && !out.empty() && !in.empty() && known / out[0] * in[0] == total)
            out[0] = in[0]; // exported for batch 1, run with a larger batch
        break;
    }
    case FLATTEN: {
        int axis = m_axis < 0 ? m_axis + (int)in.size() : m_axis;
        long long a = 1;
        for (int i = 0; i < axis; i++) a *= in[i];
        out = {(int)a, (int)(total / a)};
        break;
    }
    case SQUEEZE: {
        for (size_t i = 0; i < in.size(); i++) {
            bool drop = false;
            if (m_arg.empty())
                drop = in[i] == 1;
            for (int ax : m_arg)
                if ((ax < 0 ? ax + (int)in.size() : ax) == (int)i)
                    drop = true;
            if (!drop)
                out.push_back(in[i]);
        }
        break;
    }
    case UNSQUEEZE: {
        const int nd = (int)in.size() + (int)m_arg.size();
        out.assign(nd, 0);
        for (int ax : m_arg) out[ax < 0 ? ax + nd : ax] = 1;
        size_t k = 0;
        for (auto &o : out)
            if (o == 0)
                o = in[k++];
        break;
    }
    case IDENTITY: out = in; break;
    }
    return {out};
}

void Reshape::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *in = context->get_tensor(m_inputs_index[0]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    if (in && out && in->device && out->device && in->device != out->device) {
        espdl_copy_desc d;
        memset(&d, 0, sizeof(d));
        d.src = in->device, d.dst = out->device, d.elem_size = (int)dtype_sizeof(in->dtype), d.ndim = 1;
        d.shape[0] = in->get_size(), d.src_stride[0] = d.dst_stride[0] = 1;
        context->note(espdl_b200_copy(&d, context->stream));
    }
}

static std::vector<int> int_param(fbs::FbsModel *m, const std::string &node, int index)
{
    std::vector<int> v;
    if (TensorBase *t = m->get_operation_parameter(node, index)) {
        for (int i = 0; i < t->get_size(); i++)
            v.push_back(t->dtype == DATA_TYPE_INT64 ? (int)((int64_t *)t->data)[i] : ((int32_t *)t->data)[i]);
        delete t;
    }
    return v;
}

Module *Reshape::deserialize_reshape(fbs::FbsModel *m, std::string node)
{
    return new Reshape(RESHAPE, int_param(m, node, 1), 0, node.c_str(), node_quant(m, node));
}
Module *Reshape::deserialize_flatten(fbs::FbsModel *m, std::string node)
{
    int axis = 1;
    m->get_operation_attribute(node, "axis", axis);
    return new Reshape(FLATTEN, {}, axis, node.c_str(), node_quant(m, node));
}
Module *Reshape::deserialize_squeeze(fbs::FbsModel *m, std::string node)
{
    std::vector<int> axes = int_param(m, node, 1);
    if (axes.empty())
        m->get_operation_attribute(node, "axes", axes);
    return new Reshape(SQUEEZE, axes, 0, node.c_str(), node_quant(m, node));
}
Module *Reshape::deserialize_unsqueeze(fbs::FbsModel *m, std::string node)
{
    std::vector<int> axes = int_param(m, node, 1);
    if (axes.empty())
        m->get_operation_attribute(node, "axes", axes);
    return new Reshape(UNSQUEEZE, axes, 0, node.c_str(), node_quant(m, node));
}
Module *Reshape::deserialize_identity(fbs::FbsModel *m, std::string node)
{
    return new Reshape(IDENTITY, {}, 0, node.c_str(), node_quant(m, node));
}

// --------------------------------------------------------------------------------- softmax
Softmax::~Softmax()
{
    if (m_dev_table)
        espdl_b200_arena_free(m_dev_table);
}

void Softmax::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *in = context->get_tensor(m_inputs_index[0]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    int st = (!in || !out || !in->device || !out->device) ? ESPDL_ERR_INVALID_ARG : ESPDL_OK;
    const int nd = in ? (int)in->shape.size() : 0;
    const int ax = axis < 0 ? axis + nd : axis;
    if (!st && (in->dtype != DATA_TYPE_INT8 || ax < 0 || ax >= nd))
        st = ESPDL_ERR_UNSUPPORTED;
    if (!st)
        st = upload_exp_table(m_dev_table, m_table_exponent, (int)in->exponent);
    if (!st) {
        espdl_softmax_desc d;
        memset(&d, 0, sizeof(d));
        long long inner = 1;
        for (int i = ax + 1; i < nd; i++) inner *= in->shape[i];
        d.input = (const int8_t *)in->device, d.output = out->device, d.exp_table = (const float *)m_dev_table;
        d.len = in->shape[ax], d.rows = in->get_size() / d.len;
        d.inner = (int)inner, d.log = m_log ? 1 : 0, d.in_exponent = in->exponent;
        d.out_dtype = espdl_dtype(out), d.out_exponent = out->exponent, d.round_mode = context->round_mode;
        st = inner > INT_MAX ? ESPDL_ERR_TOO_LARGE : espdl_b200_softmax(&d, context->stream);
    }
    if (st)
        ESP_LOGE("Softmax", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

Module *Softmax::deserialize(fbs::FbsModel *m, std::string node)
{
    int axis = -1;
    m->get_operation_attribute(node, "axis", axis);
    return new Softmax(node.c_str(), axis, MODULE_NON_INPLACE, node_quant(m, node));
}

// --------------------------------------------------------------------------------- Pow
Pow::Pow(const char *name, module_inplace_t inplace, quant_type_t quant_type) : Elementwise(ESPDL_ELT_POW, name, inplace, quant_type) {}
Pow::~Pow()
{
    if (m_dev_table)
        espdl_b200_arena_free(m_dev_table);
}
Module *Pow::deserialize(fbs::FbsModel *m, std::string node) { return new Pow(node.c_str(), MODULE_NON_INPLACE, node_quant(m, node)); }

void Pow::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *a = context->get_tensor(m_inputs_index[0]), *b = context->get_tensor(m_inputs_index[1]);
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    espdl_eltwise_desc d;
    memset(&d, 0, sizeof(d));
    int st = ESPDL_OK;
    if (!a || !b || !out || !a->device || !b->device || !out->device)
        st = ESPDL_ERR_INVALID_ARG;
    if (!st && !pack_shapes(out->shape, a->shape, b->shape, d))
        st = ESPDL_ERR_UNSUPPORTED;
    if (!st && a->dtype == DATA_TYPE_INT8) {
        const int key[4] = {(int)a->exponent, (int)b->exponent, (int)out->exponent, (int)context->round_mode};
        if (!m_dev_table || memcmp(key, m_table_key, sizeof(key)) != 0) {
            // every (base, power) pair once, with the host's powf: c_impl_pow_n_n of esp-dl/dl/base/dl_base_pow.cpp:49-63
            std::vector<int8_t> table(65536);
            const float s0 = DL_SCALE(key[0]), s1 = DL_SCALE(key[1]), rescale = DL_RESCALE(key[2]);
            for (int ua = 0; ua < 256; ua++)
                for (int ub = 0; ub < 256; ub++) {
                    const float base_val = (float)(int8_t)(ua ^ 0x80) * s0, exp_val = (float)(int8_t)(ub ^ 0x80) * s1;
                    const float r = powf(base_val, exp_val) * rescale;
                    long long q;
                    if (!(fabsf(r) < 2147483520.f))
                        q = INT_MIN; // what the float -> int conversion of a NaN or an infinity gives where the reference runs
                    else
                        q = key[3] == ESPDL_ROUND_HALF_EVEN ? (long long)rintf(r) : (long long)floorf((float)((double)r + 0.5));
                    table[ua * 256 + ub] = (int8_t)std::max(-128ll, std::min(127ll, q));
                }
            if (!m_dev_table && espdl_b200_arena_alloc(table.size(), &m_dev_table) != ESPDL_OK)
                st = ESPDL_ERR_NO_MEM;
            if (!st)
                st = espdl_b200_upload(m_dev_table, table.data(), table.size(), nullptr);
            if (!st)
                st = espdl_b200_stream_sync(nullptr);
            memcpy(m_table_key, key, sizeof(key));
        }
        d.table = m_dev_table;
    }
    if (!st) {
        d.input0 = a->device, d.input1 = b->device, d.output = out->device;
        d.op = m_op, d.in_dtype = espdl_dtype(a), d.out_dtype = espdl_dtype(out);
        d.in0_exponent = a->exponent, d.in1_exponent = b->exponent, d.out_exponent = out->exponent;
        d.round_mode = context->round_mode;
        st = espdl_b200_eltwise(&d, context->stream);
    }
    if (st)
        ESP_LOGE("Pow", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

// --------------------------------------------------------------------------------- LogSoftmax, LpNormalization
Module *LogSoftmax::deserialize(fbs::FbsModel *m, std::string node)
{
    int axis = -1;
    m->get_operation_attribute(node, "axis", axis);
    return new LogSoftmax(node.c_str(), axis, MODULE_NON_INPLACE, node_quant(m, node));
}

void LpNormalization::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *x = context->get_tensor(m_inputs_index[0]);
    TensorBase *y = context->get_tensor(m_outputs_index[0]);
    int st = (!x || !y || !x->device || !y->device || x->shape.empty()) ? ESPDL_ERR_INVALID_ARG : ESPDL_OK;
    if (!st) {
        const int nd = (int)x->shape.size(), axis = m_axis < 0 ? nd + m_axis : m_axis;
        espdl_norm_desc d;
        memset(&d, 0, sizeof(d));
        if (axis < 0 || axis >= nd) {
            st = ESPDL_ERR_INVALID_ARG;
        } else {
            long long inner = 1;
            for (int i = axis + 1; i < nd; i++) inner *= x->shape[i];
            d.input = x->device, d.output = y->device, d.op = ESPDL_NORM_LP, d.dtype = quant_dtype(quant_type);
            d.len = x->shape[axis], d.rows = x->get_size() / d.len, d.inner = inner, d.p = m_p;
            d.in_exponent = x->exponent, d.out_exponent = y->exponent, d.round_mode = context->round_mode;
            st = espdl_b200_norm(&d, context->stream);
        }
    }
    if (st)
        ESP_LOGE("LpNormalization", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

Module *LpNormalization::deserialize(fbs::FbsModel *m, std::string node)
{
    int axis = -1, p = 2;
    m->get_operation_attribute(node, "axis", axis);
    m->get_operation_attribute(node, "p", p);
    return new LpNormalization(axis, p, node.c_str(), MODULE_NON_INPLACE, node_quant(m, node));
}

// --------------------------------------------------------------------------------- ReverseSequence, ScatterND
static esp_err_t upload_parameters(ModelContext *context, const std::vector<int> &inputs)
{
    for (int idx : inputs) {
        TensorBase *t = context->get_tensor(idx);
        if (t && t->data && !t->device && t->to_device() != ESP_OK) // host data and no device copy: a parameter
            return ESP_FAIL;
    }
    return espdl_b200_stream_sync(nullptr) == ESPDL_OK ? ESP_OK : ESP_FAIL;
}

esp_err_t ReverseSequence::prepare(ModelContext *context) { return upload_parameters(context, m_inputs_index); }

void ReverseSequence::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *x = context->get_tensor(m_inputs_index[0]);
    TensorBase *lens = m_inputs_index.size() > 1 ? context->get_tensor(m_inputs_index[1]) : nullptr;
    TensorBase *y = context->get_tensor(m_outputs_index[0]);
    int st = (!x || !y || !lens || !x->device || !y->device || !lens->device || x->shape.size() < 2) ? ESPDL_ERR_INVALID_ARG : ESPDL_OK;
    if (!st && (lens->dtype != DATA_TYPE_INT64 || m_batch_axis + m_time_axis != 1 || x->device == y->device ||
                lens->get_size() < x->shape[m_batch_axis]))
        st = ESPDL_ERR_UNSUPPORTED;
    if (!st) {
        espdl_reverse_sequence_desc d;
        memset(&d, 0, sizeof(d));
        d.input = x->device, d.output = y->device, d.seq_lens = (const int64_t *)lens->device;
        d.elem_size = (int)dtype_sizeof(x->dtype), d.batch_axis = m_batch_axis, d.dim0 = x->shape[0], d.dim1 = x->shape[1];
        d.feature = 1;
        for (size_t i = 2; i < x->shape.size(); i++) d.feature *= x->shape[i];
        st = espdl_b200_reverse_sequence(&d, context->stream);
    }
    if (st)
        ESP_LOGE("ReverseSequence", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

Module *ReverseSequence::deserialize(fbs::FbsModel *m, std::string node)
{
    int batch_axis = 1, time_axis = 0;
    m->get_operation_attribute(node, "batch_axis", batch_axis);
    m->get_operation_attribute(node, "time_axis", time_axis);
    // the reference swaps in place after a copy; here the kernel reads one buffer and writes another
    return new ReverseSequence(batch_axis, time_axis, node.c_str(), MODULE_NON_INPLACE, node_quant(m, node));
}

ScatterND::ScatterND(const std::string &reduction, const char *name, module_inplace_t inplace, quant_type_t quant_type) :
    Module(name, inplace, quant_type), m_reduction(ESPDL_SCATTER_NONE)
{
    // unknown strings fall back to "none", as apply_reduction does (dl_module_scatter_nd.hpp:34-47)
    for (auto &kv : std::initializer_list<std::pair<const char *, int>>{
             {"add", ESPDL_SCATTER_ADD}, {"mul", ESPDL_SCATTER_MUL}, {"max", ESPDL_SCATTER_MAX}, {"min", ESPDL_SCATTER_MIN}})
        if (reduction == kv.first)
            m_reduction = kv.second;
}

esp_err_t ScatterND::prepare(ModelContext *context) { return upload_parameters(context, m_inputs_index); }

void ScatterND::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    TensorBase *data = context->get_tensor(m_inputs_index[0]);
    TensorBase *indices = m_inputs_index.size() > 1 ? context->get_tensor(m_inputs_index[1]) : nullptr;
    TensorBase *updates = m_inputs_index.size() > 2 ? context->get_tensor(m_inputs_index[2]) : nullptr;
    TensorBase *out = context->get_tensor(m_outputs_index[0]);
    int st = (!data || !indices || !updates || !out || !data->device || !indices->device || !updates->device || !out->device ||
              indices->shape.empty() || data->shape.empty())
        ? ESPDL_ERR_INVALID_ARG
        : ESPDL_OK;
    if (!st && indices->dtype != DATA_TYPE_INT64)
        st = ESPDL_ERR_UNSUPPORTED;
    if (!st) {
        espdl_scatter_nd_desc d;
        memset(&d, 0, sizeof(d));
        const int depth = indices->shape.back(), rank = (int)data->shape.size();
        if (depth < 1 || depth > rank || depth > 6) {
            st = ESPDL_ERR_INVALID_ARG;
        } else {
            d.data = data->device, d.indices = (const int64_t *)indices->device, d.updates = updates->device, d.output = out->device;
            d.dtype = espdl_dtype(data), d.reduction = m_reduction, d.index_depth = depth;
            d.n_slices = (int)(indices->get_size() / depth);
            d.slice_size = 1;
            for (int i = depth; i < rank; i++) d.slice_size *= data->shape[i];
            d.data_size = data->get_size();
            long long stride = d.data_size;
            for (int k = 0; k < depth; k++) {
                stride /= data->shape[k];
                d.axis_offset[k] = stride;
            }
            if (updates->get_size() < (long long)d.n_slices * d.slice_size)
                st = ESPDL_ERR_INVALID_ARG;
            else
                st = espdl_b200_scatter_nd(&d, context->stream);
        }
    }
    if (st)
        ESP_LOGE("ScatterND", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

Module *ScatterND::deserialize(fbs::FbsModel *m, std::string node)
{
    std::string reduction = "none";
    m->get_operation_attribute(node, "reduction", reduction);
    return new ScatterND(reduction, node.c_str(), MODULE_INPLACE_CHANGED_BUFFER, node_quant(m, node));
}

// --------------------------------------------------------------------------------- GRU, LSTM
Rnn::~Rnn()
{
    if (m_dev_sigmoid)
        espdl_b200_arena_free(m_dev_sigmoid);
    if (m_dev_tanh)
        espdl_b200_arena_free(m_dev_tanh);
}

std::vector<std::vector<int>> Rnn::get_output_shape(std::vector<std::vector<int>> &input_shapes)
{
    // dl_module_gru.hpp:80-101, dl_module_lstm.hpp:86-112
    std::vector<std::vector<int>> out;
    if (input_shapes.size() < 3 || input_shapes[0].size() < 3)
        return out;
    const std::vector<int> &x = input_shapes[0];
    const int seq = m_layout == 0 ? x[0] : x[1], batch = m_layout == 0 ? x[1] : x[0];
    out.push_back({seq, m_direction_num, batch, m_hidden_size});
    out.push_back({m_direction_num, batch, m_hidden_size});
    if (m_op == ESPDL_RNN_LSTM)
        out.push_back({m_direction_num, batch, m_hidden_size});
    return out;
}

// math::sigmoid / math::tanh and the two tables of esp-dl/dl/math/include/dl_math.hpp:168-176, 324-429
static float rnn_sigmoid(float x) { return (float)(1.0 / (1.0 + expf(-x))); }
static float rnn_tanh(float x) { return 2 * rnn_sigmoid(2 * x) - 1; }
static int rnn_table(int gate_exponent, bool tanh_table, std::vector<float> &table)
{
    const float bound = tanh_table ? (float)3.5 : (float)6.3, input_scale = DL_SCALE(gate_exponent);
    int quant_min = (int)(-bound / input_scale) - 1, quant_max = (int)(bound / input_scale) + 1;
    if (-quant_min > quant_max)
        quant_max = -quant_min;
    table.resize((size_t)quant_max + 1);
    for (int i = 0; i <= quant_max; i++) table[i] = tanh_table ? rnn_tanh(i * input_scale) : rnn_sigmoid(i * input_scale);
    return quant_max;
}

esp_err_t Rnn::prepare(ModelContext *context)
{
    if (m_gate_exponent > 0 || m_gate_exponent < -14) // the tables would be empty or hold millions of entries
        return ESP_FAIL;
    for (int which = 0; which < 2; which++) {
        std::vector<float> table;
        const int mx = rnn_table(m_gate_exponent, which == 1, table);
        void *&dev = which ? m_dev_tanh : m_dev_sigmoid;
        (which ? m_tanh_max : m_sigmoid_max) = mx;
        if (!dev && espdl_b200_arena_alloc(table.size() * sizeof(float), &dev) != ESPDL_OK)
            return ESP_FAIL;
        if (espdl_b200_upload(dev, table.data(), table.size() * sizeof(float), nullptr) != ESPDL_OK)
            return ESP_FAIL;
    }
    return upload_parameters(context, m_inputs_index);
}

void Rnn::forward(ModelContext *context, runtime_mode_t mode)
{
    (void)mode;
    auto in = [&](size_t i) { return m_inputs_index.size() > i ? context->get_tensor(m_inputs_index[i]) : nullptr; };
    auto out = [&](size_t i) { return m_outputs_index.size() > i ? context->get_tensor(m_outputs_index[i]) : nullptr; };
    TensorBase *x = in(0), *w = in(1), *r = in(2), *b = in(3), *h0 = in(5), *c0 = m_op == ESPDL_RNN_LSTM ? in(6) : nullptr;
    TensorBase *y = out(0), *yh = out(1), *yc = m_op == ESPDL_RNN_LSTM ? out(2) : nullptr;
    int st = (!x || !w || !r || !y || !yh || !x->device || !w->device || !r->device || !y->device || !yh->device || x->shape.size() != 3)
        ? ESPDL_ERR_INVALID_ARG
        : ESPDL_OK;
    if (!st && ((b && !b->device) || (h0 && !h0->device) || (c0 && !c0->device) || (yc && !yc->device)))
        st = ESPDL_ERR_INVALID_ARG;
    if (!st) {
        const int G = m_op == ESPDL_RNN_GRU ? 3 : 4, H = m_hidden_size;
        const int seq = m_layout == 0 ? x->shape[0] : x->shape[1], batch = m_layout == 0 ? x->shape[1] : x->shape[0], isz = x->shape[2];
        // what the reference supports (dl_module_gru.hpp:161, dl_module_lstm.hpp:179): one sequence at a time; the weights'
        // shapes as its first step checks them; an int16 bias at the gates' exponent; an int16 cell state at that exponent
        const bool shapes_ok = batch == 1 && w->shape == std::vector<int>({m_direction_num, G * H, isz}) &&
            r->shape == std::vector<int>({m_direction_num, G * H, H}) && (!b || (b->dtype == DATA_TYPE_INT16 && b->get_size() >= m_direction_num * 2 * G * H)) &&
            (!h0 || h0->get_size() >= m_direction_num * H) && (!c0 || (c0->dtype == DATA_TYPE_INT16 && c0->get_size() >= m_direction_num * H)) &&
            (!yc || (yc->dtype == DATA_TYPE_INT16 && (int)yc->exponent == m_gate_exponent));
        if (!shapes_ok || x->dtype != w->dtype || x->dtype != r->dtype || y->dtype != x->dtype || yh->dtype != x->dtype || (h0 && h0->dtype != x->dtype)) {
            st = ESPDL_ERR_UNSUPPORTED;
        } else {
            espdl_rnn_desc d;
            memset(&d, 0, sizeof(d));
            d.x = x->device, d.w = w->device, d.r = r->device, d.b = b ? (const int16_t *)b->device : nullptr;
            d.initial_h = h0 ? h0->device : nullptr, d.initial_c = c0 ? (const int16_t *)c0->device : nullptr;
            d.y = y->device, d.y_h = yh->device, d.y_c = yc ? (int16_t *)yc->device : nullptr;
            d.sigmoid_table = (const float *)m_dev_sigmoid, d.tanh_table = (const float *)m_dev_tanh;
            d.sigmoid_max = m_sigmoid_max, d.tanh_max = m_tanh_max;
            d.op = m_op, d.dtype = quant_dtype(quant_type), d.seq_length = seq, d.input_size = isz, d.hidden_size = H, d.directions = m_direction_num;
            d.x_exponent = x->exponent, d.w_exponent = w->exponent, d.r_exponent = r->exponent, d.h_exponent = yh->exponent;
            d.y_exponent = y->exponent, d.c_exponent = yc ? (int)yc->exponent : m_gate_exponent, d.gate_exponent = m_gate_exponent;
            d.round_mode = context->round_mode;
            st = espdl_b200_rnn(&d, context->stream);
        }
    }
    if (st)
        ESP_LOGE("Rnn", "%s failed: %s", name ? name : "?", espdl_b200_strerror(st));
    context->note(st);
}

static Module *deserialize_rnn(fbs::FbsModel *m, const std::string &node, bool lstm)
{
    int hidden_size = 0, layout = 0, gate_exponent = -8, flag = lstm ? 0 : 0;
    std::string direction = "forward";
    m->get_operation_attribute(node, "hidden_size", hidden_size);
    m->get_operation_attribute(node, "direction", direction);
    m->get_operation_attribute(node, "layout", layout);
    m->get_operation_attribute(node, "gate_exponent", gate_exponent);
    m->get_operation_attribute(node, lstm ? "input_forget" : "linear_before_reset", flag);
    // dl_module_gru.hpp:409-412: only the PyTorch form (linear_before_reset = 1); dl_module_lstm.hpp:480-483: no coupled gates
    if ((!lstm && flag == 0) || (lstm && flag == 1) || hidden_size <= 0)
        return nullptr;
    const int dirs = direction == "bidirectional" ? 2 : 1;
    if (lstm)
        return new LSTM(node.c_str(), hidden_size, dirs, layout, gate_exponent, MODULE_NON_INPLACE, node_quant(m, node));
    return new GRU(node.c_str(), hidden_size, dirs, layout, gate_exponent, MODULE_NON_INPLACE, node_quant(m, node));
}
Module *GRU::deserialize(fbs::FbsModel *m, std::string node) { return deserialize_rnn(m, node, false); }
Module *LSTM::deserialize(fbs::FbsModel *m, std::string node) { return deserialize_rnn(m, node, true); }

// --------------------------------------------------------------------------------- registry
void ModuleCreator::register_dl_modules()
{
    if (registered)
        return;
    registered = true;
    // same op-type strings as the reference registry (esp-dl/dl/module/include/dl_module_creator.hpp:134-204)
    register_module("Conv", Conv::deserialize);
    register_module("Gemm", Gemm::deserialize);
    register_module("MatMul", MatMul::deserialize);
    register_module("Add", Add::deserialize);
    register_module("Sub", Sub::deserialize);
    register_module("Mul", Mul::deserialize);
    register_module("Max", Max::deserialize);
    register_module("Min", Min::deserialize);
    register_module("Div", Div::deserialize);
    register_module("Mod", Mod::deserialize);
    register_module("Greater", Greater::deserialize);
    register_module("GreaterOrEqual", GreaterOrEqual::deserialize);
    register_module("Equal", Equal::deserialize);
    register_module("Less", Less::deserialize);
    register_module("LessOrEqual", LessOrEqual::deserialize);
    register_module("RequantizeLinear", RequantizeLinear::deserialize);
    register_module("QuantizeLinear", RequantizeLinear::deserialize);
    register_module("DequantizeLinear", RequantizeLinear::deserialize);
    for (const char *op : {"LUT", "Swish", "Sigmoid", "Tanh", "HardSwish", "HardSigmoid", "Gelu", "Elu", "LeakyRelu", "Exp", "Log", "Sqrt",
                           "Neg", "Abs"})
        register_module(op, LUT::deserialize);
    for (const char *op : {"ReduceMean", "ReduceSum", "ReduceMax", "ReduceMin", "ReduceL1", "ReduceSumSquare", "ReduceL2", "ReduceProd",
                           "ReduceLogSum", "ReduceLogSumExp"})
        register_module(op, Reduce::deserialize);
    register_module("Pow", Pow::deserialize);
    register_module("LogSoftmax", LogSoftmax::deserialize);
    register_module("LpNormalization", LpNormalization::deserialize);
    register_module("ReverseSequence", ReverseSequence::deserialize);
    register_module("ScatterND", ScatterND::deserialize);
    register_module("GRU", GRU::deserialize);
    register_module("LSTM", LSTM::deserialize);
    register_module("Slice", Slice::deserialize);
    register_module("Pad", Pad::deserialize);
    register_module("Clip", Clip::deserialize);
    register_module("Relu", Relu::deserialize);
    register_module("PRelu", PRelu::deserialize);
    register_module("MaxPool", MaxPool::deserialize);
    register_module("AveragePool", AveragePool::deserialize);
    register_module("GlobalAveragePool", GlobalAveragePool::deserialize);
    register_module("Resize", Resize::deserialize);
    register_module("Concat", Concat::deserialize);
    register_module("Split", Split::deserialize);
    register_module("Transpose", Transpose::deserialize);
    register_module("SpaceToDepth", SpaceToDepth::deserialize);
    register_module("DepthToSpace", DepthToSpace::deserialize);
    register_module("Gather", Gather::deserialize);
    register_module("InsertZeros", InsertZeros::deserialize);
    register_module("StreamingCache", StreamingCache::deserialize);
    register_module("RMSNormalization", RMSNormalization::deserialize);
    register_module("LayerNormalization", LayerNormalization::deserialize);
    register_module("Reshape", Reshape::deserialize_reshape);
    register_module("Flatten", Reshape::deserialize_flatten);
    register_module("Squeeze", Reshape::deserialize_squeeze);
    register_module("Unsqueeze", Reshape::deserialize_unsqueeze);
    register_module("Identity", Reshape::deserialize_identity);
    register_module("Softmax", Softmax::deserialize);
}

} // namespace module
} // namespace dl
