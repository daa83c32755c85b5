// dl::TensorBase and dl::ExponentInfo for the B200 backend.
// Same public fields and meaning as the reference (esp-dl/dl/tensor/include/dl_tensor_base.hpp:22-211,297-744):
// shape, dtype, power-of-two exponent (per tensor, or per output channel for filters), and a 16-byte
// aligned `data` pointer on the HOST.  Added for this backend: `device`, the address of the tensor's
// copy in HBM (activations live in the model's device arena; parameters are uploaded once at load).
#pragma once
#include "dl_define.hpp"
#include <string>
#include <vector>

namespace dl {

class ExponentInfo {
    int m_exponent;
    std::vector<int> m_exponents;

public:
    ExponentInfo(int exponent = 0) : m_exponent(exponent) {}
    ExponentInfo(const std::vector<int> &exponents) : m_exponent(0)
    {
        if (exponents.size() <= 1)
            m_exponent = exponents.empty() ? 0 : exponents[0];
        else
            m_exponents = exponents;
    }
    bool is_per_channel() const { return !m_exponents.empty(); }
    int size() const { return m_exponents.empty() ? 1 : (int)m_exponents.size(); }
    int get(int i = 0) const { return m_exponents.empty() ? m_exponent : m_exponents[i]; }
    const std::vector<int> &values() const { return m_exponents; }
    operator int() const { return m_exponent; }
    bool operator==(const ExponentInfo &o) const { return m_exponent == o.m_exponent && m_exponents == o.m_exponents; }
    bool operator!=(const ExponentInfo &o) const { return !(*this == o); }
};

typedef enum {
    DATA_TYPE_UNDEFINED = 0,
    DATA_TYPE_FLOAT = 1,
    DATA_TYPE_UINT8 = 2,
    DATA_TYPE_INT8 = 3,
    DATA_TYPE_UINT16 = 4,
    DATA_TYPE_INT16 = 5,
    DATA_TYPE_INT32 = 6,
    DATA_TYPE_INT64 = 7,
    DATA_TYPE_STRING = 8,
    DATA_TYPE_BOOL = 9,
    DATA_TYPE_FLOAT16 = 10,
    DATA_TYPE_DOUBLE = 11,
    DATA_TYPE_UINT32 = 12,
    DATA_TYPE_UINT64 = 13,
} dtype_t;

size_t dtype_sizeof(dtype_t dtype);
const char *dtype_to_string(dtype_t dtype);
const char *quant_type_to_string(quant_type_t type);
const char *activation_type_to_string(activation_type_t type);
std::string vector_to_string(const std::vector<int> &v);

class TensorBase {
public:
    int size;               ///< number of elements
    std::vector<int> shape; ///< shape
    dtype_t dtype;
    ExponentInfo exponent;
    bool auto_free;         ///< `data` is owned by this object
    std::vector<int> axis_offset;
    void *data;             ///< host copy (may be null for arena intermediates)
    void *device;           ///< device copy (null until the tensor is placed / uploaded)
    bool device_owned;      ///< `device` was allocated by this object (parameters)
    int row_stride = 0;     ///< device copy only: elements between consecutive rows of the last axis when this tensor
                            ///< is a channel slice of a wider one (the arena planner's Concat / Split views); 0 = dense
    uint32_t caps;

    TensorBase(std::vector<int> shape, const void *element, int exponent = 0, dtype_t dtype = DATA_TYPE_FLOAT, bool deep = true,
               uint32_t caps = MALLOC_CAP_DEFAULT);
    TensorBase(std::vector<int> shape, const void *element, const std::vector<int> &exponents, dtype_t dtype = DATA_TYPE_FLOAT,
               bool deep = true, uint32_t caps = MALLOC_CAP_DEFAULT);
    virtual ~TensorBase();
    TensorBase(const TensorBase &) = delete;
    TensorBase &operator=(const TensorBase &) = delete;

    int get_size() const { return size; }
    size_t get_bytes() const { return (size_t)size * dtype_sizeof(dtype); }
    size_t get_aligned_bytes() const { return (get_bytes() + 15) & ~(size_t)15; }
    std::vector<int> get_shape() const { return shape; }
    TensorBase &set_shape(const std::vector<int> &s);
    dtype_t get_dtype() const { return dtype; }
    int get_exponent() const { return exponent; }
    void *get_element_ptr() { return data; }
    template <typename T> T *get_element_ptr() { return (T *)data; }
    template <typename T> T get_element(int index) { return ((T *)data)[index]; }

    /// Copy / quantise / dequantise / requantise `tensor` into this one on the host, with the reference's
    /// arithmetic (esp-dl/dl/tensor/src/dl_tensor_base.cpp:223-404).  Used for user-supplied inputs.
    bool assign(TensorBase *tensor);
    /// Exact comparison used by Model::test (int8 exact, int16 within +-1, float within 1e-4 relative).
    bool equal(TensorBase *tensor, float epsilon = 2e-5f, bool verbose = false);
    /// Upload `data` to a freshly allocated device buffer (parameters).
    esp_err_t to_device(void *stream = nullptr);
    void print(bool print_data = false);

private:
    void init(const void *element, bool deep);
};

} // namespace dl
