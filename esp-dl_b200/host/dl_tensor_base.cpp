#include "dl_tensor_base.hpp"
#include "espdl_b200.h"

#include <cmath>
#include <cstdarg>
#include <cstring>

namespace dl {

void log_message(char level, const char *tag, const char *fmt, ...)
{
    static const char *verbose = getenv("ESPDL_B200_VERBOSE");
    if (level != 'E' && !verbose)
        return;
    fprintf(stderr, "%c (%s) ", level, tag);
    va_list ap;
    va_start(ap, fmt);
    vfprintf(stderr, fmt, ap);
    va_end(ap);
    fputc('\n', stderr);
}

size_t dtype_sizeof(dtype_t dtype)
{
    switch (dtype) {
    case DATA_TYPE_FLOAT: case DATA_TYPE_INT32: case DATA_TYPE_UINT32: return 4;
    case DATA_TYPE_INT8: case DATA_TYPE_UINT8: case DATA_TYPE_BOOL: return 1;
    case DATA_TYPE_INT16: case DATA_TYPE_UINT16: case DATA_TYPE_FLOAT16: return 2;
    case DATA_TYPE_INT64: case DATA_TYPE_UINT64: case DATA_TYPE_DOUBLE: return 8;
    default: return 0;
    }
}

const char *dtype_to_string(dtype_t dtype)
{
    switch (dtype) {
    case DATA_TYPE_FLOAT: return "float";
    case DATA_TYPE_INT8: return "int8";
    case DATA_TYPE_UINT8: return "uint8";
    case DATA_TYPE_INT16: return "int16";
    case DATA_TYPE_UINT16: return "uint16";
    case DATA_TYPE_INT32: return "int32";
    case DATA_TYPE_INT64: return "int64";
    case DATA_TYPE_DOUBLE: return "double";
    case DATA_TYPE_BOOL: return "bool";
    default: return "undefined";
    }
}

const char *quant_type_to_string(quant_type_t type)
{
    switch (type) {
    case QUANT_TYPE_FLOAT32: return "F32";
    case QUANT_TYPE_SYMM_8BIT: return "S8";
    case QUANT_TYPE_SYMM_16BIT: return "S16";
    case QUANT_TYPE_SYMM_32BIT: return "S32";
    default: return "NONE";
    }
}

const char *activation_type_to_string(activation_type_t type)
{
    switch (type) {
    case Linear: return "Linear";
    case ReLU: return "ReLU";
    case LeakyReLU: return "LeakyReLU";
    case PReLU: return "PReLU";
    }
    return "";
}

std::string vector_to_string(const std::vector<int> &v)
{
    std::string s = "[";
    for (size_t i = 0; i < v.size(); i++) s += std::to_string(v[i]) + (i + 1 < v.size() ? ", " : "");
    return s + "]";
}

void TensorBase::init(const void *element, bool deep)
{
    size = 1;
    for (int d : shape) size *= d;
    axis_offset.assign(shape.size(), 1);
    for (int i = (int)shape.size() - 2; i >= 0; i--) axis_offset[i] = axis_offset[i + 1] * shape[i + 1];
    device = nullptr;
    device_owned = false;
    if (deep) {
        size_t bytes = get_aligned_bytes();
        data = nullptr;
        if (posix_memalign(&data, 64, bytes ? bytes : 16))
            data = nullptr;
        auto_free = true;
        if (data) {
            if (element)
                memcpy(data, element, get_bytes());
            else
                memset(data, 0, bytes);
        }
    } else {
        data = const_cast<void *>(element);
        auto_free = false;
    }
}

TensorBase::TensorBase(std::vector<int> shape, const void *element, int exponent, dtype_t dtype, bool deep, uint32_t caps) :
    shape(shape), dtype(dtype), exponent(exponent), caps(caps)
{
    init(element, deep);
}

TensorBase::TensorBase(std::vector<int> shape, const void *element, const std::vector<int> &exponents, dtype_t dtype, bool deep,
                       uint32_t caps) :
    shape(shape), dtype(dtype), exponent(exponents), caps(caps)
{
    init(element, deep);
}

TensorBase::~TensorBase()
{
    if (auto_free && data)
        free(data);
    if (device_owned && device)
        espdl_b200_arena_free(device);
}

TensorBase &TensorBase::set_shape(const std::vector<int> &s)
{
    shape = s;
    axis_offset.assign(shape.size(), 1);
    for (int i = (int)shape.size() - 2; i >= 0; i--) axis_offset[i] = axis_offset[i + 1] * shape[i + 1];
    return *this;
}

esp_err_t TensorBase::to_device(void *stream)
{
    if (!data)
        return ESP_FAIL;
    if (!device) {
        if (espdl_b200_arena_alloc(get_aligned_bytes(), &device) != ESPDL_OK)
            return ESP_FAIL;
        device_owned = true;
    }
    return espdl_b200_upload(device, data, get_bytes(), stream) == ESPDL_OK ? ESP_OK : ESP_FAIL;
}

// dl::tool::round for the generic targets: (int)floorf(value + 0.5) with a double literal
// (esp-dl/dl/tool/src/dl_tool.cpp:72-75).
static inline int round_half_up(float v) { return (int)floorf((float)((double)v + 0.5)); }

template <typename RT> static RT quantize(float input, float inv_scale)
{
    int out = round_half_up(input * inv_scale);
    const int lo = sizeof(RT) == 1 ? -128 : -32768, hi = sizeof(RT) == 1 ? 127 : 32767;
    return (RT)(out < lo ? lo : (out > hi ? hi : out));
}

template <typename DT, typename ST> static void requant_loop(DT *dst, const ST *src, int n, float src_scale, float inv_scale)
{
    for (int i = 0; i < n; i++) dst[i] = quantize<DT>((float)src[i] * src_scale, inv_scale);
}

bool TensorBase::assign(TensorBase *t)
{
    if (!t || t->get_size() != get_size() || !data || !t->data)
        return false;
    if (exponent.is_per_channel() || t->exponent.is_per_channel()) {
        if (exponent == t->exponent && dtype == t->dtype) {
            memcpy(data, t->data, get_bytes());
            return true;
        }
        return false;
    }
    const int n = get_size();
    if (exponent == t->exponent && dtype == t->dtype) {
        memcpy(data, t->data, get_bytes());
    } else if (t->dtype == DATA_TYPE_FLOAT) {
        const float inv = DL_RESCALE((int)exponent);
        const float *s = (const float *)t->data;
        if (dtype == DATA_TYPE_INT8)
            for (int i = 0; i < n; i++) ((int8_t *)data)[i] = quantize<int8_t>(s[i], inv);
        else if (dtype == DATA_TYPE_INT16)
            for (int i = 0; i < n; i++) ((int16_t *)data)[i] = quantize<int16_t>(s[i], inv);
        else
            return false;
    } else if (dtype == DATA_TYPE_FLOAT) {
        const float sc = DL_SCALE((int)t->exponent);
        if (t->dtype == DATA_TYPE_INT8)
            for (int i = 0; i < n; i++) ((float *)data)[i] = (float)((int8_t *)t->data)[i] * sc;
        else if (t->dtype == DATA_TYPE_INT16)
            for (int i = 0; i < n; i++) ((float *)data)[i] = (float)((int16_t *)t->data)[i] * sc;
        else
            return false;
    } else if (exponent == t->exponent) {
        if (dtype == DATA_TYPE_INT8 && t->dtype == DATA_TYPE_INT16) {
            for (int i = 0; i < n; i++) {
                int v = ((int16_t *)t->data)[i];
                ((int8_t *)data)[i] = (int8_t)(v < -128 ? -128 : (v > 127 ? 127 : v));
            }
        } else if (dtype == DATA_TYPE_INT16 && t->dtype == DATA_TYPE_INT8) {
            for (int i = 0; i < n; i++) ((int16_t *)data)[i] = ((int8_t *)t->data)[i];
        } else {
            return false;
        }
    } else {
        const float src_scale = DL_SCALE((int)t->exponent);
        const float inv = (float)(1.0 / (double)DL_SCALE((int)exponent));
        if (dtype == DATA_TYPE_INT8 && t->dtype == DATA_TYPE_INT8)
            requant_loop((int8_t *)data, (const int8_t *)t->data, n, src_scale, inv);
        else if (dtype == DATA_TYPE_INT16 && t->dtype == DATA_TYPE_INT16)
            requant_loop((int16_t *)data, (const int16_t *)t->data, n, src_scale, inv);
        else if (dtype == DATA_TYPE_INT8 && t->dtype == DATA_TYPE_INT16)
            requant_loop((int8_t *)data, (const int16_t *)t->data, n, src_scale, inv);
        else if (dtype == DATA_TYPE_INT16 && t->dtype == DATA_TYPE_INT8)
            requant_loop((int16_t *)data, (const int8_t *)t->data, n, src_scale, inv);
        else
            return false;
    }
    return true;
}

bool TensorBase::equal(TensorBase *t, float epsilon, bool verbose)
{
    if (!t || t->get_size() != get_size() || t->dtype != dtype || !data || !t->data)
        return false;
    const int n = get_size();
    int bad = -1;
    if (dtype == DATA_TYPE_INT8) {
        for (int i = 0; i < n && bad < 0; i++)
            if (((int8_t *)data)[i] != ((int8_t *)t->data)[i])
                bad = i;
    } else if (dtype == DATA_TYPE_INT16) { // the reference tolerates one code on 16-bit outputs
        for (int i = 0; i < n && bad < 0; i++)
            if (abs(((int16_t *)data)[i] - ((int16_t *)t->data)[i]) > 1)
                bad = i;
    } else if (dtype == DATA_TYPE_FLOAT) {
        for (int i = 0; i < n && bad < 0; i++) {
            float a = ((float *)data)[i], b = ((float *)t->data)[i];
            if (fabsf(a - b) > epsilon + 1e-4f * fabsf(b))
                bad = i;
        }
    } else {
        return memcmp(data, t->data, get_bytes()) == 0;
    }
    if (bad >= 0 && verbose)
        ESP_LOGE("TensorBase", "first mismatch at element %d", bad);
    return bad < 0;
}

void TensorBase::print(bool print_data)
{
    fprintf(stderr, "TensorBase shape %s dtype %s exponent %d size %d\n", vector_to_string(shape).c_str(), dtype_to_string(dtype),
            (int)exponent, size);
    if (print_data && data && dtype == DATA_TYPE_INT8) {
        for (int i = 0; i < size && i < 64; i++) fprintf(stderr, "%d ", ((int8_t *)data)[i]);
        fputc('\n', stderr);
    }
}

} // namespace dl
