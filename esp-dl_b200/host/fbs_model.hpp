// Reader of the `.espdl` model container and of the FlatBuffers graph inside it.
//
// The reference ships this layer only as a header (esp-dl/fbs_loader/include/fbs_model.hpp:23-424) plus a
// prebuilt library; this is an independent implementation of that contract written against the schema
// (esp-dl/fbs_loader/espdl.fbs) and the container comments in esp-dl/fbs_loader/include/fbs_loader.hpp:13-97:
//   EDL1  "EDL1" | u32 mode | u32 size | flatbuffer
//   EDL2  "EDL2" | u32 mode | u32 size | u32 pad | flatbuffer                       (16-byte aligned payload)
//   PDL1/PDL2  magic | u32 n | n x (u32 data_off, u32 name_off, u32 name_len) | names | EDL1/EDL2 models
//   PDL3  "PDL3" | char version[16] | u32 package_size | u8 sha256[32] | u32 n | table as PDL2
// Encrypted payloads (mode 1, AES-128-CTR) are rejected: no key handling is implemented here.
#pragma once
#include "dl_tensor_base.hpp"

#include <map>
#include <string>
#include <vector>

namespace fbs {

typedef enum {
    MODEL_LOCATION_IN_FLASH_RODATA = 0, ///< the argument is the address of the model bytes in memory
    MODEL_LOCATION_IN_FLASH_PARTITION = 1,
    MODEL_LOCATION_IN_SDCARD = 2, ///< the argument is a file path
} model_location_type_t;

class FbsModel {
public:
    /// `data` points at the FlatBuffer (container header already stripped).  With `auto_free` the model owns it.
    FbsModel(const void *data, size_t size, model_location_type_t location, bool encrypt, bool rodata_move, bool auto_free,
             bool param_copy);
    ~FbsModel();

    std::vector<std::string> topological_sort();
    esp_err_t get_operation_attribute(std::string node_name, std::string attribute_name, int &ret_value);
    esp_err_t get_operation_attribute(std::string node_name, std::string attribute_name, float &ret_value);
    esp_err_t get_operation_attribute(std::string node_name, std::string attribute_name, std::string &ret_value);
    esp_err_t get_operation_attribute(std::string node_name, std::string attribute_name, std::vector<int> &ret_value);
    esp_err_t get_operation_attribute(std::string node_name, std::string attribute_name, std::vector<float> &ret_value);
    esp_err_t get_operation_attribute(std::string node_name, std::string attribute_name, dl::quant_type_t &ret_value);
    esp_err_t get_operation_attribute(std::string node_name, std::string attribute_name, dl::activation_type_t &ret_value);
    esp_err_t get_operation_attribute(std::string node_name, std::string attribute_name, dl::resize_mode_t &ret_value);
    esp_err_t get_operation_inputs_and_outputs(std::string node_name, std::vector<std::string> &inputs,
                                               std::vector<std::string> &outputs);
    std::string get_operation_type(std::string node_name);
    /// New TensorBase (caller owns) for input `index` of the node if it is an initializer, else nullptr.
    /// The payload is deep-copied when `m_param_copy`, otherwise it aliases the model bytes.
    dl::TensorBase *get_operation_parameter(std::string node_name, int index = 1, uint32_t caps = MALLOC_CAP_DEFAULT);
    dl::TensorBase *get_operation_lut(std::string node_name, uint32_t caps = MALLOC_CAP_DEFAULT, std::string attribute_name = "lut");
    bool is_parameter(std::string name);
    const void *get_tensor_raw_data(std::string tensor_name);
    dl::dtype_t get_tensor_dtype(std::string tensor_name);
    std::vector<int> get_tensor_shape(std::string tensor_name);
    std::vector<int> get_tensor_exponents(std::string tensor_name);
    dl::dtype_t get_value_info_dtype(std::string var_name);
    std::vector<int> get_value_info_shape(std::string var_name);
    int get_value_info_exponent(std::string var_name);
    dl::TensorBase *get_test_input_tensor(std::string tensor_name);
    dl::TensorBase *get_test_output_tensor(std::string tensor_name);
    std::vector<std::string> get_test_outputs_name();
    std::vector<std::string> get_graph_inputs();
    std::vector<std::string> get_graph_outputs();
    void clear_map();
    void load_map();
    std::string get_model_name();
    int64_t get_model_version();
    std::string get_model_doc_string();
    std::string get_model_metadata_prop(const std::string &key);
    size_t get_size() const { return m_size; }
    /// false when an offset or a length of the FlatBuffer points outside it (checked once, when the model is constructed)
    bool valid() const { return m_valid; }
    void print();

    bool m_param_copy;

private:
    dl::TensorBase *tensor_from_table(const void *tensor_table, bool copy);
    const void *find_attribute(const std::string &node, const std::string &attr);
    model_location_type_t m_location;
    bool m_auto_free;
    size_t m_size;
    bool m_valid = false;
    const uint8_t *m_data;
    std::map<std::string, const void *> m_name_to_node_map;
    std::map<std::string, const void *> m_name_to_initial_tensor_map;
    std::map<std::string, const void *> m_name_to_value_info_map;
    std::map<std::string, const void *> m_name_to_test_inputs_value_map;
    std::map<std::string, const void *> m_name_to_test_outputs_value_map;
    std::vector<std::string> m_node_order;
};

class FbsLoader {
public:
    /// `name` is a file path (MODEL_LOCATION_IN_SDCARD) or the address of the model bytes in memory.
    FbsLoader(const char *name = nullptr, model_location_type_t location = MODEL_LOCATION_IN_FLASH_RODATA);
    ~FbsLoader();
    FbsModel *load(const int model_index = 0, const uint8_t *key = nullptr, bool param_copy = true);
    FbsModel *load(const char *model_name, const uint8_t *key = nullptr, bool param_copy = true);
    FbsModel *load(const uint8_t *key = nullptr, bool param_copy = true) { return load(0, key, param_copy); }
    int get_model_num();
    void list_models();
    const char *get_model_location_string();
    /// PDL3 packages (magic, version[16], package_size, sha256[32], model table): the header fields and the
    /// integrity check of fbs_loader.hpp:195-262.  The digest covers bytes [0, package_size) with the 32 bytes of
    /// the stored digest taken as zeros.
    bool is_pdl3() const { return m_pdl3; }
    esp_err_t get_package_version(char *out_version, size_t out_size);
    uint32_t get_package_size();
    esp_err_t get_package_sha256(uint8_t out_sha256[32]);
    esp_err_t calc_package_sha256(uint8_t out_sha256[32]);
    bool verify_package_sha256();

private:
    FbsModel *make(size_t offset, const uint8_t *key, bool param_copy);
    bool m_pdl3 = false;
    int m_header_bytes = 16; ///< per-model header: 12 bytes in EDL1 / PDL1 containers, 16 in the others
    std::vector<uint8_t> m_file; ///< file contents when loaded from a path
    const uint8_t *m_buf = nullptr;
    size_t m_buf_size = 0; ///< 0 = unknown (in-memory model)
    model_location_type_t m_location;
    std::vector<std::pair<std::string, size_t>> m_models; ///< (name, byte offset of the EDLx header)
};

} // namespace fbs
