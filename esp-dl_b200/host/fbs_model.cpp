#include "fbs_model.hpp"

#include "fbs_crypto.hpp"

#include <cstring>
#include <fstream>
#include <set>

namespace fbs {
namespace {

// Minimal FlatBuffers table access (little-endian host).  Field ids are the declaration order in espdl.fbs.
struct Table {
    const uint8_t *p = nullptr;
    Table() {}
    explicit Table(const uint8_t *ptr) : p(ptr) {}
    explicit operator bool() const { return p != nullptr; }
    template <typename T> static T rd(const uint8_t *q)
    {
        T v;
        memcpy(&v, q, sizeof(T));
        return v;
    }
    uint16_t off(int fid) const
    {
        const uint8_t *vt = p - rd<int32_t>(p);
        const uint16_t vt_size = rd<uint16_t>(vt);
        const int o = 4 + 2 * fid;
        return o + 2 <= vt_size ? rd<uint16_t>(vt + o) : 0;
    }
    template <typename T> T scalar(int fid, T def = 0) const
    {
        const uint16_t o = off(fid);
        return o ? rd<T>(p + o) : def;
    }
    const uint8_t *indirect(int fid) const
    {
        const uint16_t o = off(fid);
        if (!o)
            return nullptr;
        const uint8_t *q = p + o;
        return q + rd<uint32_t>(q);
    }
    const uint8_t *inline_struct(int fid) const
    {
        const uint16_t o = off(fid);
        return o ? p + o : nullptr;
    }
    Table table(int fid) const { return Table(indirect(fid)); }
    std::string str(int fid) const
    {
        const uint8_t *q = indirect(fid);
        return q ? std::string((const char *)q + 4, rd<uint32_t>(q)) : std::string();
    }
    uint32_t vec_len(int fid) const
    {
        const uint8_t *q = indirect(fid);
        return q ? rd<uint32_t>(q) : 0;
    }
    const uint8_t *vec_data(int fid) const
    {
        const uint8_t *q = indirect(fid);
        return q ? q + 4 : nullptr;
    }
    Table vec_table(int fid, uint32_t i) const
    {
        const uint8_t *q = vec_data(fid) + 4 * i;
        return Table(q + rd<uint32_t>(q));
    }
    std::string vec_str(int fid, uint32_t i) const
    {
        const uint8_t *q = vec_data(fid) + 4 * i;
        const uint8_t *s = q + rd<uint32_t>(q);
        return std::string((const char *)s + 4, rd<uint32_t>(s));
    }
};

// field ids (esp-dl/fbs_loader/espdl.fbs)
enum { MODEL_MODEL_VERSION = 5, MODEL_DOC_STRING = 6, MODEL_GRAPH = 7, MODEL_METADATA = 8 };
enum { GRAPH_NODE = 0, GRAPH_NAME = 1, GRAPH_INITIALIZER = 2, GRAPH_INPUT = 4, GRAPH_OUTPUT = 5, GRAPH_VALUE_INFO = 6,
       GRAPH_TEST_INPUTS = 8, GRAPH_TEST_OUTPUTS = 9 };
enum { NODE_INPUT = 0, NODE_OUTPUT = 1, NODE_NAME = 2, NODE_OP_TYPE = 3, NODE_ATTRIBUTE = 5 };
enum { ATTR_NAME = 0, ATTR_TYPE = 3, ATTR_F = 4, ATTR_I = 5, ATTR_S = 6, ATTR_T = 7, ATTR_FLOATS = 10, ATTR_INTS = 11 };
enum { TENSOR_DIMS = 0, TENSOR_DATA_TYPE = 1, TENSOR_FLOAT_DATA = 2, TENSOR_INT32_DATA = 3, TENSOR_INT64_DATA = 5, TENSOR_NAME = 6,
       TENSOR_RAW_DATA = 8, TENSOR_EXPONENTS = 13 };
enum { VI_NAME = 0, VI_TYPE = 1, VI_EXPONENTS = 3 };
enum { TI_VALUE_TYPE = 0, TI_VALUE = 1 };
enum { TT_ELEM_TYPE = 0, TT_SHAPE = 1 };
enum { AT_FLOAT = 1, AT_INT = 2, AT_STRING = 3, AT_TENSOR = 4, AT_FLOATS = 6, AT_INTS = 7 };

Table root_of(const uint8_t *data) { return Table(data + Table::rd<uint32_t>(data)); }
Table graph_of(const uint8_t *data) { return root_of(data).table(MODEL_GRAPH); }

std::vector<int> read_i64_vec(const Table &t, int fid)
{
    std::vector<int> v;
    const uint32_t n = t.vec_len(fid);
    const uint8_t *d = t.vec_data(fid);
    for (uint32_t i = 0; i < n; i++) v.push_back((int)Table::rd<int64_t>(d + 8 * i));
    return v;
}

// Walks everything the accessors below can touch, once, with every offset and length checked against the buffer: a
// truncated or damaged file is refused when it is loaded instead of being read out of bounds later.
struct Verifier {
    const uint8_t *lo;
    size_t size;
    bool ok = true;
    bool in(const uint8_t *q, size_t n)
    {
        if (!ok || q < lo || n > size || (size_t)(q - lo) > size - n) {
            ok = false;
        }
        return ok;
    }
    // a table: its vtable lies inside the buffer, and so does the table's inline part
    bool table(const uint8_t *t)
    {
        if (!in(t, 4))
            return false;
        const int64_t vt_off = (int64_t)(t - lo) - (int64_t)Table::rd<int32_t>(t);
        if (vt_off < 0 || (uint64_t)vt_off + 4 > size)
            return ok = false;
        const uint8_t *vt = lo + vt_off;
        const uint16_t vt_size = Table::rd<uint16_t>(vt), t_size = Table::rd<uint16_t>(vt + 2);
        return vt_size >= 4 && vt_size % 2 == 0 && in(vt, vt_size) && in(t, t_size < 4 ? 4 : t_size);
    }
    // offset of field `fid` inside a verified table (0 = absent); `width` bytes at that place are inside the table
    uint16_t field(const uint8_t *t, int fid, size_t width)
    {
        const uint8_t *vt = t - Table::rd<int32_t>(t);
        const uint16_t vt_size = Table::rd<uint16_t>(vt), t_size = Table::rd<uint16_t>(vt + 2);
        const int o = 4 + 2 * fid;
        if (o + 2 > vt_size)
            return 0;
        const uint16_t f = Table::rd<uint16_t>(vt + o);
        if (f && (size_t)f + width > (size_t)(t_size < 4 ? 4 : t_size)) {
            ok = false;
        }
        return ok ? f : 0;
    }
    const uint8_t *indirect(const uint8_t *t, int fid)
    {
        const uint16_t f = field(t, fid, 4);
        if (!f)
            return nullptr;
        const uint8_t *q = t + f;
        const uint32_t rel = Table::rd<uint32_t>(q);
        const uint8_t *r = q + rel;
        return in(r, 4) ? r : nullptr;
    }
    // a vector of `elem`-byte scalars (a string with elem = 1); returns the element count
    uint32_t vec(const uint8_t *t, int fid, size_t elem)
    {
        const uint8_t *r = indirect(t, fid);
        if (!r)
            return 0;
        const uint32_t n = Table::rd<uint32_t>(r);
        return in(r + 4, (size_t)n * elem) ? n : 0;
    }
    // a vector of offsets to tables / strings: calls `each` on every target that lies inside the buffer
    template <typename F> void vec_of(const uint8_t *t, int fid, F each)
    {
        const uint8_t *r = indirect(t, fid);
        if (!r)
            return;
        const uint32_t n = Table::rd<uint32_t>(r);
        if (!in(r + 4, (size_t)n * 4))
            return;
        for (uint32_t i = 0; i < n && ok; i++) {
            const uint8_t *q = r + 4 + 4 * (size_t)i;
            const uint8_t *target = q + Table::rd<uint32_t>(q);
            if (in(target, 4))
                each(target);
        }
    }
    void string_at(const uint8_t *sp) { in(sp + 4, Table::rd<uint32_t>(sp)); }
    void sub_table(const uint8_t *t, int fid, void (Verifier::*walk)(const uint8_t *))
    {
        const uint8_t *r = indirect(t, fid);
        if (r && table(r))
            (this->*walk)(r);
    }
    void tensor(const uint8_t *t)
    {
        vec(t, TENSOR_NAME, 1);
        const uint32_t nd = vec(t, TENSOR_DIMS, 8);
        const uint16_t dtf = field(t, TENSOR_DATA_TYPE, 4);
        const size_t raw = 16 * (size_t)vec(t, TENSOR_RAW_DATA, 16); // a vector of 16-byte AlignedBytes structs (espdl.fbs)
        const size_t f32 = vec(t, TENSOR_FLOAT_DATA, 4), i32 = vec(t, TENSOR_INT32_DATA, 4), i64 = vec(t, TENSOR_INT64_DATA, 8);
        vec(t, TENSOR_EXPONENTS, 8);
        if (!ok)
            return;
        // the payload holds what the dims promise (a tensor object is built over it and read to its end)
        const uint8_t *dims = nd ? indirect(t, TENSOR_DIMS) + 4 : nullptr;
        uint64_t count = 1;
        for (uint32_t i = 0; i < nd; i++) {
            const int64_t d = Table::rd<int64_t>(dims + 8 * (size_t)i);
            if (d < 0 || d > 0x7fffffff || (count *= (uint64_t)d) > 0x7fffffffull)
                ok = false;
        }
        const size_t have = raw ? raw : (f32 ? 4 * f32 : (i32 ? 4 * i32 : 8 * i64));
        const size_t es = dl::dtype_sizeof((dl::dtype_t)(dtf ? Table::rd<int32_t>(t + dtf) : 0));
        if (ok && have && es && count * es > have) {
            ok = false;
        }
    }
    void dimension_value(const uint8_t *t) { field(t, 1, 8); }
    void dimension(const uint8_t *t) { sub_table(t, 0, &Verifier::dimension_value); }
    void shape(const uint8_t *t)
    {
        vec_of(t, 0, [&](const uint8_t *d) {
            if (table(d))
                dimension(d);
        });
    }
    void tensor_type(const uint8_t *t)
    {
        field(t, TT_ELEM_TYPE, 4);
        sub_table(t, TT_SHAPE, &Verifier::shape);
    }
    void type_info(const uint8_t *t)
    {
        field(t, TI_VALUE_TYPE, 1);
        sub_table(t, TI_VALUE, &Verifier::tensor_type);
    }
    void value_info(const uint8_t *t)
    {
        vec(t, VI_NAME, 1);
        sub_table(t, VI_TYPE, &Verifier::type_info);
        vec(t, VI_EXPONENTS, 8);
    }
    void attribute(const uint8_t *t)
    {
        vec(t, ATTR_NAME, 1);
        field(t, ATTR_TYPE, 4);
        field(t, ATTR_F, 4);
        field(t, ATTR_I, 8);
        vec(t, ATTR_S, 1);
        sub_table(t, ATTR_T, &Verifier::tensor);
        vec(t, ATTR_FLOATS, 4);
        vec(t, ATTR_INTS, 8);
    }
    void node(const uint8_t *t)
    {
        vec(t, NODE_NAME, 1);
        vec(t, NODE_OP_TYPE, 1);
        for (int fid : {NODE_INPUT, NODE_OUTPUT}) vec_of(t, fid, [&](const uint8_t *sp) { string_at(sp); });
        vec_of(t, NODE_ATTRIBUTE, [&](const uint8_t *a) {
            if (table(a))
                attribute(a);
        });
    }
    void graph(const uint8_t *g)
    {
        vec(g, GRAPH_NAME, 1);
        vec_of(g, GRAPH_NODE, [&](const uint8_t *n) {
            if (table(n))
                node(n);
        });
        for (int fid : {GRAPH_INITIALIZER, GRAPH_TEST_INPUTS, GRAPH_TEST_OUTPUTS})
            vec_of(g, fid, [&](const uint8_t *t) {
                if (table(t))
                    tensor(t);
            });
        for (int fid : {GRAPH_INPUT, GRAPH_OUTPUT, GRAPH_VALUE_INFO})
            vec_of(g, fid, [&](const uint8_t *v) {
                if (table(v))
                    value_info(v);
            });
    }
    bool model()
    {
        if (size < 8 || !in(lo, 4))
            return false;
        const uint8_t *root = lo + Table::rd<uint32_t>(lo);
        if (!table(root))
            return false;
        field(root, MODEL_MODEL_VERSION, 8);
        vec(root, MODEL_DOC_STRING, 1);
        vec_of(root, MODEL_METADATA, [&](const uint8_t *kv) {
            if (table(kv)) {
                vec(kv, 0, 1);
                vec(kv, 1, 1);
            }
        });
        sub_table(root, MODEL_GRAPH, &Verifier::graph);
        return ok;
    }
};

} // namespace

FbsModel::FbsModel(const void *data, size_t size, model_location_type_t location, bool encrypt, bool rodata_move, bool auto_free,
                   bool param_copy) :
    m_param_copy(param_copy), m_location(location), m_auto_free(auto_free), m_size(size), m_data((const uint8_t *)data)
{
    (void)encrypt;
    (void)rodata_move;
    Verifier v{m_data, m_size};
    m_valid = m_data && m_size && v.model();
    if (m_valid)
        load_map();
    else
        ESP_LOGE("FbsModel", "the model's FlatBuffer is truncated or damaged: an offset or a length points outside its %zu bytes", m_size);
}

FbsModel::~FbsModel()
{
    if (m_auto_free)
        free(const_cast<uint8_t *>(m_data));
}

void FbsModel::clear_map()
{
    m_name_to_node_map.clear();
    m_name_to_initial_tensor_map.clear();
    m_name_to_value_info_map.clear();
    m_name_to_test_inputs_value_map.clear();
    m_name_to_test_outputs_value_map.clear();
    m_node_order.clear();
}

void FbsModel::load_map()
{
    clear_map();
    Table g = graph_of(m_data);
    for (uint32_t i = 0; i < g.vec_len(GRAPH_NODE); i++) {
        Table n = g.vec_table(GRAPH_NODE, i);
        m_name_to_node_map[n.str(NODE_NAME)] = n.p;
        m_node_order.push_back(n.str(NODE_NAME));
    }
    for (uint32_t i = 0; i < g.vec_len(GRAPH_INITIALIZER); i++) {
        Table t = g.vec_table(GRAPH_INITIALIZER, i);
        m_name_to_initial_tensor_map[t.str(TENSOR_NAME)] = t.p;
    }
    for (int fid : {GRAPH_INPUT, GRAPH_OUTPUT, GRAPH_VALUE_INFO})
        for (uint32_t i = 0; i < g.vec_len(fid); i++) {
            Table v = g.vec_table(fid, i);
            m_name_to_value_info_map[v.str(VI_NAME)] = v.p;
        }
    for (uint32_t i = 0; i < g.vec_len(GRAPH_TEST_INPUTS); i++) {
        Table t = g.vec_table(GRAPH_TEST_INPUTS, i);
        m_name_to_test_inputs_value_map[t.str(TENSOR_NAME)] = t.p;
    }
    for (uint32_t i = 0; i < g.vec_len(GRAPH_TEST_OUTPUTS); i++) {
        Table t = g.vec_table(GRAPH_TEST_OUTPUTS, i);
        m_name_to_test_outputs_value_map[t.str(TENSOR_NAME)] = t.p;
    }
}

// Kahn's algorithm over tensor names; ties keep the file order, which is already a valid order for exported models.
std::vector<std::string> FbsModel::topological_sort()
{
    std::set<std::string> ready;
    for (auto &kv : m_name_to_initial_tensor_map) ready.insert(kv.first);
    for (auto &n : get_graph_inputs()) ready.insert(n);
    std::vector<std::string> order, pending = m_node_order;
    while (!pending.empty()) {
        std::vector<std::string> next;
        bool progress = false;
        for (auto &name : pending) {
            std::vector<std::string> ins, outs;
            get_operation_inputs_and_outputs(name, ins, outs);
            bool ok = true;
            for (auto &i : ins)
                if (!i.empty() && !ready.count(i))
                    ok = false;
            if (ok) {
                order.push_back(name);
                for (auto &o : outs) ready.insert(o);
                progress = true;
            } else {
                next.push_back(name);
            }
        }
        if (!progress) {
            ESP_LOGE("FbsModel", "graph has a cycle or a dangling input; %d nodes unscheduled", (int)next.size());
            break;
        }
        pending.swap(next);
    }
    return order;
}

const void *FbsModel::find_attribute(const std::string &node, const std::string &attr)
{
    auto it = m_name_to_node_map.find(node);
    if (it == m_name_to_node_map.end())
        return nullptr;
    Table n((const uint8_t *)it->second);
    for (uint32_t i = 0; i < n.vec_len(NODE_ATTRIBUTE); i++) {
        Table a = n.vec_table(NODE_ATTRIBUTE, i);
        if (a.str(ATTR_NAME) == attr)
            return a.p;
    }
    return nullptr;
}

esp_err_t FbsModel::get_operation_attribute(std::string node_name, std::string attribute_name, int &ret_value)
{
    Table a((const uint8_t *)find_attribute(node_name, attribute_name));
    if (!a || a.scalar<int32_t>(ATTR_TYPE) != AT_INT || !a.inline_struct(ATTR_I))
        return ESP_FAIL;
    ret_value = (int)Table::rd<int64_t>(a.inline_struct(ATTR_I));
    return ESP_OK;
}

esp_err_t FbsModel::get_operation_attribute(std::string node_name, std::string attribute_name, float &ret_value)
{
    Table a((const uint8_t *)find_attribute(node_name, attribute_name));
    if (!a || a.scalar<int32_t>(ATTR_TYPE) != AT_FLOAT || !a.inline_struct(ATTR_F))
        return ESP_FAIL;
    ret_value = Table::rd<float>(a.inline_struct(ATTR_F));
    return ESP_OK;
}

esp_err_t FbsModel::get_operation_attribute(std::string node_name, std::string attribute_name, std::string &ret_value)
{
    Table a((const uint8_t *)find_attribute(node_name, attribute_name));
    if (!a || a.scalar<int32_t>(ATTR_TYPE) != AT_STRING)
        return ESP_FAIL;
    ret_value = std::string((const char *)a.vec_data(ATTR_S), a.vec_len(ATTR_S));
    return ESP_OK;
}

esp_err_t FbsModel::get_operation_attribute(std::string node_name, std::string attribute_name, std::vector<int> &ret_value)
{
    Table a((const uint8_t *)find_attribute(node_name, attribute_name));
    if (!a || a.scalar<int32_t>(ATTR_TYPE) != AT_INTS)
        return ESP_FAIL;
    ret_value = read_i64_vec(a, ATTR_INTS);
    return ESP_OK;
}

esp_err_t FbsModel::get_operation_attribute(std::string node_name, std::string attribute_name, std::vector<float> &ret_value)
{
    Table a((const uint8_t *)find_attribute(node_name, attribute_name));
    if (!a || a.scalar<int32_t>(ATTR_TYPE) != AT_FLOATS)
        return ESP_FAIL;
    ret_value.clear();
    for (uint32_t i = 0; i < a.vec_len(ATTR_FLOATS); i++) ret_value.push_back(Table::rd<float>(a.vec_data(ATTR_FLOATS) + 4 * i));
    return ESP_OK;
}

esp_err_t FbsModel::get_operation_attribute(std::string node_name, std::string attribute_name, dl::quant_type_t &ret_value)
{
    std::string s;
    if (get_operation_attribute(node_name, attribute_name, s) != ESP_OK)
        return ESP_FAIL;
    if (s == "S8")
        ret_value = dl::QUANT_TYPE_SYMM_8BIT;
    else if (s == "S16")
        ret_value = dl::QUANT_TYPE_SYMM_16BIT;
    else if (s == "F32")
        ret_value = dl::QUANT_TYPE_FLOAT32;
    else
        ret_value = dl::QUANT_TYPE_NONE;
    return ESP_OK;
}

esp_err_t FbsModel::get_operation_attribute(std::string node_name, std::string attribute_name, dl::activation_type_t &ret_value)
{
    std::string s;
    if (get_operation_attribute(node_name, attribute_name, s) != ESP_OK)
        return ESP_FAIL;
    if (s == "Relu" || s == "ReLU")
        ret_value = dl::ReLU;
    else if (s == "LeakyRelu")
        ret_value = dl::LeakyReLU;
    else if (s == "PRelu")
        ret_value = dl::PReLU;
    else
        ret_value = dl::Linear;
    return ESP_OK;
}

esp_err_t FbsModel::get_operation_attribute(std::string node_name, std::string attribute_name, dl::resize_mode_t &ret_value)
{
    std::string s;
    if (get_operation_attribute(node_name, attribute_name, s) != ESP_OK)
        return ESP_FAIL;
    ret_value = s == "linear" ? dl::RESIZE_LINEAR : (s == "cubic" ? dl::RESIZE_CUBIC : dl::RESIZE_NEAREST);
    return ESP_OK;
}

esp_err_t FbsModel::get_operation_inputs_and_outputs(std::string node_name, std::vector<std::string> &inputs,
                                                     std::vector<std::string> &outputs)
{
    auto it = m_name_to_node_map.find(node_name);
    if (it == m_name_to_node_map.end())
        return ESP_FAIL;
    Table n((const uint8_t *)it->second);
    inputs.clear();
    outputs.clear();
    for (uint32_t i = 0; i < n.vec_len(NODE_INPUT); i++) inputs.push_back(n.vec_str(NODE_INPUT, i));
    for (uint32_t i = 0; i < n.vec_len(NODE_OUTPUT); i++) outputs.push_back(n.vec_str(NODE_OUTPUT, i));
    return ESP_OK;
}

std::string FbsModel::get_operation_type(std::string node_name)
{
    auto it = m_name_to_node_map.find(node_name);
    return it == m_name_to_node_map.end() ? std::string() : Table((const uint8_t *)it->second).str(NODE_OP_TYPE);
}

dl::TensorBase *FbsModel::tensor_from_table(const void *tensor_table, bool copy)
{
    Table t((const uint8_t *)tensor_table);
    std::vector<int> dims = read_i64_vec(t, TENSOR_DIMS);
    const dl::dtype_t dt = (dl::dtype_t)t.scalar<int32_t>(TENSOR_DATA_TYPE);
    std::vector<int> exps = read_i64_vec(t, TENSOR_EXPONENTS);
    const void *payload = t.vec_data(TENSOR_RAW_DATA);
    if (!payload) {
        for (int fid : {TENSOR_FLOAT_DATA, TENSOR_INT32_DATA, TENSOR_INT64_DATA})
            if (t.vec_len(fid)) {
                payload = t.vec_data(fid);
                break;
            }
    }
    if (dims.empty())
        dims = {1};
    if (exps.size() > 1)
        return new dl::TensorBase(dims, payload, exps, dt, copy);
    return new dl::TensorBase(dims, payload, exps.empty() ? 0 : exps[0], dt, copy);
}

dl::TensorBase *FbsModel::get_operation_parameter(std::string node_name, int index, uint32_t caps)
{
    (void)caps;
    std::vector<std::string> ins, outs;
    if (get_operation_inputs_and_outputs(node_name, ins, outs) != ESP_OK || index >= (int)ins.size())
        return nullptr;
    auto it = m_name_to_initial_tensor_map.find(ins[index]);
    if (it == m_name_to_initial_tensor_map.end())
        return nullptr;
    return tensor_from_table(it->second, m_param_copy);
}

dl::TensorBase *FbsModel::get_operation_lut(std::string node_name, uint32_t caps, std::string attribute_name)
{
    (void)caps;
    std::string lut_name;
    if (get_operation_attribute(node_name, attribute_name, lut_name) != ESP_OK)
        return nullptr;
    auto it = m_name_to_initial_tensor_map.find(lut_name);
    if (it == m_name_to_initial_tensor_map.end())
        return nullptr;
    return tensor_from_table(it->second, m_param_copy);
}

bool FbsModel::is_parameter(std::string name) { return m_name_to_initial_tensor_map.count(name) != 0; }

const void *FbsModel::get_tensor_raw_data(std::string tensor_name)
{
    auto it = m_name_to_initial_tensor_map.find(tensor_name);
    return it == m_name_to_initial_tensor_map.end() ? nullptr : Table((const uint8_t *)it->second).vec_data(TENSOR_RAW_DATA);
}

dl::dtype_t FbsModel::get_tensor_dtype(std::string tensor_name)
{
    auto it = m_name_to_initial_tensor_map.find(tensor_name);
    return it == m_name_to_initial_tensor_map.end() ? dl::DATA_TYPE_UNDEFINED
                                                    : (dl::dtype_t)Table((const uint8_t *)it->second).scalar<int32_t>(TENSOR_DATA_TYPE);
}

std::vector<int> FbsModel::get_tensor_shape(std::string tensor_name)
{
    auto it = m_name_to_initial_tensor_map.find(tensor_name);
    return it == m_name_to_initial_tensor_map.end() ? std::vector<int>() : read_i64_vec(Table((const uint8_t *)it->second), TENSOR_DIMS);
}

std::vector<int> FbsModel::get_tensor_exponents(std::string tensor_name)
{
    auto it = m_name_to_initial_tensor_map.find(tensor_name);
    return it == m_name_to_initial_tensor_map.end() ? std::vector<int>()
                                                    : read_i64_vec(Table((const uint8_t *)it->second), TENSOR_EXPONENTS);
}

dl::dtype_t FbsModel::get_value_info_dtype(std::string var_name)
{
    auto it = m_name_to_value_info_map.find(var_name);
    if (it == m_name_to_value_info_map.end())
        return dl::DATA_TYPE_UNDEFINED;
    Table ti = Table((const uint8_t *)it->second).table(VI_TYPE);
    if (!ti || ti.scalar<uint8_t>(TI_VALUE_TYPE) != 1)
        return dl::DATA_TYPE_UNDEFINED;
    return (dl::dtype_t)ti.table(TI_VALUE).scalar<int32_t>(TT_ELEM_TYPE);
}

std::vector<int> FbsModel::get_value_info_shape(std::string var_name)
{
    std::vector<int> shape;
    auto it = m_name_to_value_info_map.find(var_name);
    if (it == m_name_to_value_info_map.end())
        return shape;
    Table ti = Table((const uint8_t *)it->second).table(VI_TYPE);
    if (!ti || ti.scalar<uint8_t>(TI_VALUE_TYPE) != 1)
        return shape;
    Table sh = ti.table(TI_VALUE).table(TT_SHAPE);
    if (!sh)
        return shape;
    for (uint32_t i = 0; i < sh.vec_len(0); i++) {
        Table dv = sh.vec_table(0, i).table(0);
        shape.push_back(dv ? (int)dv.scalar<int64_t>(1) : -1);
    }
    return shape;
}

int FbsModel::get_value_info_exponent(std::string var_name)
{
    auto it = m_name_to_value_info_map.find(var_name);
    if (it == m_name_to_value_info_map.end())
        return 0;
    std::vector<int> e = read_i64_vec(Table((const uint8_t *)it->second), VI_EXPONENTS);
    return e.empty() ? 0 : e[0];
}

dl::TensorBase *FbsModel::get_test_input_tensor(std::string tensor_name)
{
    auto it = m_name_to_test_inputs_value_map.find(tensor_name);
    return it == m_name_to_test_inputs_value_map.end() ? nullptr : tensor_from_table(it->second, true);
}

dl::TensorBase *FbsModel::get_test_output_tensor(std::string tensor_name)
{
    auto it = m_name_to_test_outputs_value_map.find(tensor_name);
    return it == m_name_to_test_outputs_value_map.end() ? nullptr : tensor_from_table(it->second, true);
}

std::vector<std::string> FbsModel::get_test_outputs_name()
{
    std::vector<std::string> names;
    for (auto &kv : m_name_to_test_outputs_value_map) names.push_back(kv.first);
    return names;
}

std::vector<std::string> FbsModel::get_graph_inputs()
{
    std::vector<std::string> names;
    Table g = graph_of(m_data);
    for (uint32_t i = 0; i < g.vec_len(GRAPH_INPUT); i++) names.push_back(g.vec_table(GRAPH_INPUT, i).str(VI_NAME));
    return names;
}

std::vector<std::string> FbsModel::get_graph_outputs()
{
    std::vector<std::string> names;
    Table g = graph_of(m_data);
    for (uint32_t i = 0; i < g.vec_len(GRAPH_OUTPUT); i++) names.push_back(g.vec_table(GRAPH_OUTPUT, i).str(VI_NAME));
    return names;
}

std::string FbsModel::get_model_name() { return graph_of(m_data).str(GRAPH_NAME); }
int64_t FbsModel::get_model_version() { return root_of(m_data).scalar<int64_t>(MODEL_MODEL_VERSION); }
std::string FbsModel::get_model_doc_string() { return root_of(m_data).str(MODEL_DOC_STRING); }

std::string FbsModel::get_model_metadata_prop(const std::string &key)
{
    Table r = root_of(m_data);
    for (uint32_t i = 0; i < r.vec_len(MODEL_METADATA); i++) {
        Table kv = r.vec_table(MODEL_METADATA, i);
        if (kv.str(0) == key)
            return kv.str(1);
    }
    return std::string();
}

void FbsModel::print()
{
    for (auto &name : m_node_order) fprintf(stderr, "%s: %s\n", get_operation_type(name).c_str(), name.c_str());
}

// ----------------------------------------------------------------------------- loader
FbsLoader::FbsLoader(const char *name, model_location_type_t location) : m_location(location)
{
    if (!name)
        return;
    if (location == MODEL_LOCATION_IN_SDCARD) {
        std::ifstream f(name, std::ios::binary);
        if (!f) {
            ESP_LOGE("FbsLoader", "Failed to open %s.", name);
            return;
        }
        m_file.assign(std::istreambuf_iterator<char>(f), std::istreambuf_iterator<char>());
        m_buf = m_file.data();
        m_buf_size = m_file.size();
    } else {
        m_buf = (const uint8_t *)name;
    }
    if (!m_buf || (m_buf_size && m_buf_size < 16)) {
        m_buf = nullptr;
        return;
    }
    // a buffer in memory comes without its length (as in the reference); a file's length bounds every header field
    auto inside = [&](uint64_t o, uint64_t n) { return !m_buf_size || (n <= m_buf_size && o <= m_buf_size - n); };
    auto u32 = [&](size_t o) { return Table::rd<uint32_t>(m_buf + o); };
    const std::string magic((const char *)m_buf, 4);
    // 12-byte model headers in the EDL1 / PDL1 containers, 16-byte ones in the others (fbs_loader.cpp:297-301)
    m_header_bytes = (magic == "EDL1" || magic == "PDL1") ? 12 : 16;
    if (magic == "EDL1" || magic == "EDL2") {
        m_models.push_back({"", 0});
    } else if (magic == "PDL1" || magic == "PDL2" || magic == "PDL3") {
        m_pdl3 = magic == "PDL3";
        size_t o = m_pdl3 ? 4 + 16 + 4 + 32 : 4;
        bool good = inside(o, 4);
        const uint32_t n = good ? u32(o) : 0;
        o += 4;
        good = good && inside(o, (uint64_t)n * 12);
        for (uint32_t i = 0; i < n && good; i++, o += 12) {
            const uint32_t data_off = u32(o), name_off = u32(o + 4), name_len = u32(o + 8);
            good = inside(name_off, name_len) && inside(data_off, 16) && name_len < 4096;
            if (good)
                m_models.push_back({std::string((const char *)m_buf + name_off, name_len), data_off});
        }
        if (!good) {
            ESP_LOGE("FbsLoader", "the package's model table points outside the file");
            m_models.clear();
            m_buf = nullptr;
        }
    } else {
        ESP_LOGE("FbsLoader", "unknown model container magic");
        m_buf = nullptr;
    }
}

FbsLoader::~FbsLoader() {}

int FbsLoader::get_model_num() { return (int)m_models.size(); }

void FbsLoader::list_models()
{
    for (size_t i = 0; i < m_models.size(); i++) fprintf(stderr, "model %d: %s\n", (int)i, m_models[i].first.c_str());
}

const char *FbsLoader::get_model_location_string()
{
    return m_location == MODEL_LOCATION_IN_SDCARD ? "file" : "memory";
}

esp_err_t FbsLoader::get_package_version(char *out_version, size_t out_size)
{
    if (!out_version || out_size < 16)
        return ESP_FAIL;
    if (!m_pdl3 || !m_buf)
        return ESP_FAIL;
    memcpy(out_version, m_buf + 4, 16);
    out_version[15] = '\0';
    return ESP_OK;
}

uint32_t FbsLoader::get_package_size() { return m_pdl3 && m_buf ? Table::rd<uint32_t>(m_buf + 20) : 0; }

esp_err_t FbsLoader::get_package_sha256(uint8_t out_sha256[32])
{
    if (!out_sha256 || !m_pdl3 || !m_buf)
        return ESP_FAIL;
    memcpy(out_sha256, m_buf + 24, 32);
    return ESP_OK;
}

esp_err_t FbsLoader::calc_package_sha256(uint8_t out_sha256[32])
{
    if (!out_sha256 || !m_pdl3 || !m_buf)
        return ESP_FAIL;
    const uint32_t package_size = get_package_size();
    if (package_size <= 24 + 32 || (m_buf_size && package_size > m_buf_size))
        return ESP_FAIL;
    const uint8_t zeros[32] = {0};
    Sha256 h;
    h.update(m_buf, 24);                 // magic, version, package_size
    h.update(zeros, 32);                 // the digest field counts as zeros
    h.update(m_buf + 56, package_size - 56);
    h.finish(out_sha256);
    return ESP_OK;
}

bool FbsLoader::verify_package_sha256()
{
    uint8_t stored[32], fresh[32];
    return get_package_sha256(stored) == ESP_OK && calc_package_sha256(fresh) == ESP_OK && memcmp(stored, fresh, 32) == 0;
}

FbsModel *FbsLoader::make(size_t offset, const uint8_t *key, bool param_copy)
{
    if (!m_buf)
        return nullptr;
    if (m_buf_size && (offset > m_buf_size || m_buf_size - offset < 16)) {
        ESP_LOGE("FbsLoader", "model header is truncated");
        return nullptr;
    }
    const uint8_t *h = m_buf + offset;
    const bool v1 = m_header_bytes == 12;
    const uint32_t mode = Table::rd<uint32_t>(h + 4), size = Table::rd<uint32_t>(h + 8);
    if (mode != 0 && !key) {
        ESP_LOGE("FbsLoader", "This is a cryptographic model, please enter the secret key!"); // fbs_loader.cpp:311-315
        return nullptr;
    }
    if (mode == 0 && key)
        ESP_LOGW("FbsLoader", "This is not a cryptographic model, the secret key is ignored.");
    const uint8_t *payload = h + (v1 ? 12 : 16);
    if (m_buf_size && (uint64_t)offset + (v1 ? 12 : 16) + size > m_buf_size) {
        ESP_LOGE("FbsLoader", "model payload is truncated");
        return nullptr;
    }
    // The FbsModel gets its own 16-byte aligned copy, so it may outlive the loader.
    void *copy = nullptr;
    if (posix_memalign(&copy, 64, size ? size : 16))
        return nullptr;
    if (mode != 0) {
        // AES-128-CTR with the fixed counter block 10 11 .. 1F (fbs_loader.cpp:86-124)
        const uint8_t nonce[16] = {0x10, 0x11, 0x12, 0x13, 0x14, 0x15, 0x16, 0x17, 0x18, 0x19, 0x1A, 0x1B, 0x1C, 0x1D, 0x1E, 0x1F};
        aes128_ctr(payload, (uint8_t *)copy, size, key, nonce);
    } else {
        memcpy(copy, payload, size);
    }
    // A FlatBuffer starts with the offset of its root table, which starts with the distance back to its vtable: reject
    // bytes that cannot be one (a wrong key, a damaged file) before anything walks them.
    bool sane = size >= 16;
    if (sane) {
        const uint32_t root = Table::rd<uint32_t>((const uint8_t *)copy);
        sane = root >= 4 && root % 4 == 0 && (uint64_t)root + 4 <= size;
        if (sane) {
            const int64_t vt = (int64_t)root - (int64_t)Table::rd<int32_t>((const uint8_t *)copy + root);
            sane = vt >= 4 && vt % 2 == 0 && vt + 4 <= (int64_t)size;
            if (sane) {
                const uint16_t vt_size = Table::rd<uint16_t>((const uint8_t *)copy + vt);
                sane = vt_size >= 4 && vt_size % 2 == 0 && vt + vt_size <= (int64_t)size;
            }
        }
    }
    if (!sane) {
        ESP_LOGE("FbsLoader", "%s", mode != 0 ? "the payload does not decrypt to a model: wrong key?" : "the payload is not a FlatBuffers model");
        free(copy);
        return nullptr;
    }
    FbsModel *model = new FbsModel(copy, size, m_location, mode != 0, false, true, param_copy);
    if (!model->valid()) { // the constructor has said why
        delete model;
        return nullptr;
    }
    return model;
}

FbsModel *FbsLoader::load(const int model_index, const uint8_t *key, bool param_copy)
{
    if (model_index < 0 || model_index >= (int)m_models.size())
        return nullptr;
    return make(m_models[model_index].second, key, param_copy);
}

FbsModel *FbsLoader::load(const char *model_name, const uint8_t *key, bool param_copy)
{
    for (auto &m : m_models)
        if (model_name && m.first == model_name)
            return make(m.second, key, param_copy);
    ESP_LOGE("FbsLoader", "Model %s is not found.", model_name ? model_name : "(null)");
    return nullptr;
}

} // namespace fbs
