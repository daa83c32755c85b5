// dl::module::Module, dl::module::ModuleCreator and dl::ModelContext for the B200 backend.
//
// Same plugin interface as the reference (esp-dl/dl/module/include/dl_module_base.hpp:25-140,
// esp-dl/dl/module/include/dl_module_creator.hpp:82-227): a Module is created from a graph node by a
// registered `deserialize` function, reports its output shapes, and `forward(context, mode)` runs it.
// Here forward() fills one of the C-ABI descriptors (include/espdl_b200.h) with the tensors' DEVICE
// addresses and enqueues the kernel on the context's stream; nothing is computed on the host.
#pragma once
#include "dl_tensor_base.hpp"
#include "fbs_model.hpp"

#include <functional>
#include <map>
#include <string>
#include <vector>

namespace dl {

typedef enum {
    MODULE_NON_INPLACE = 0,
    MODULE_INPLACE_UNCHANGED_BUFFER = 1, ///< output aliases the input buffer, data untouched (Reshape, Flatten, ...)
    MODULE_INPLACE_CHANGED_BUFFER = 2    ///< output may overwrite an input buffer (Add, LUT, RequantizeLinear, ...)
} module_inplace_t;

/// Tensor table of a model plus the execution state the modules need
/// (reference: esp-dl/dl/model/include/dl_model_context.hpp:13-240).
class ModelContext {
public:
    std::vector<TensorBase *> m_variables;
    std::map<std::string, int> m_name2index;
    void *stream = nullptr;        ///< CUDA stream every module enqueues on
    round_mode_t round_mode = ROUND_HALF_UP;
    int status = 0;                ///< first non-zero C-ABI status seen during forward
    void *workspace = nullptr;     ///< shared scratch for kernels that need it (int16 limb planes)
    size_t workspace_bytes = 0;
    bool own_tensors = false;

    ~ModelContext();
    int push_back_tensor(TensorBase *t, const std::string &name = "");
    TensorBase *get_tensor(int index) { return index >= 0 && index < (int)m_variables.size() ? m_variables[index] : nullptr; }
    TensorBase *get_tensor(const std::string &name);
    int get_tensor_index(const std::string &name);
    void note(int st)
    {
        if (st && !status)
            status = st;
    }
};

namespace module {

class Module {
public:
    char *name;
    module_inplace_t inplace;
    quant_type_t quant_type;
    std::vector<int> m_inputs_index;
    std::vector<int> m_outputs_index;

    Module(const char *name = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE, quant_type_t quant_type = QUANT_TYPE_NONE);
    virtual ~Module();

    virtual std::vector<int> get_outputs_index() { return m_outputs_index; }
    virtual std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) = 0;
    virtual void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) = 0;
    virtual void forward_args(void *args) { (void)args; }
    /// Called once after the tensor table is complete and parameters are on the device.
    virtual esp_err_t prepare(ModelContext *context) { (void)context; return ESP_OK; }
    /// May input `i` / output `o` be a channel slice of a wider tensor (TensorBase::row_stride != 0)?  The planner asks
    /// with the shapes of all inputs, parameters included; slices start and stride on 16-byte boundaries.
    virtual bool strided_input_ok(int i, const std::vector<std::vector<int>> &input_shapes) const
    {
        (void)i, (void)input_shapes;
        return false;
    }
    virtual bool strided_output_ok(int o, const std::vector<std::vector<int>> &input_shapes) const
    {
        (void)o, (void)input_shapes;
        return false;
    }
    /// Bytes of shared scratch forward() needs (0 for most modules).
    virtual size_t workspace_bytes(ModelContext *context) { (void)context; return 0; }
    virtual void print() {}
    virtual void reset() {}
    /// Run stand-alone on device-resident tensors (inputs/outputs must have `device` set).
    virtual void run(TensorBase *input, TensorBase *output, runtime_mode_t mode = RUNTIME_MODE_SINGLE_CORE);
    virtual void run(std::vector<TensorBase *> inputs, std::vector<TensorBase *> outputs, runtime_mode_t mode = RUNTIME_MODE_SINGLE_CORE);
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name)
    {
        (void)fbs_model;
        (void)node_name;
        return nullptr;
    }
};

class ModuleCreator {
public:
    using Creator = std::function<Module *(fbs::FbsModel *, std::string)>;
    static ModuleCreator *get_instance()
    {
        static ModuleCreator instance;
        return &instance;
    }
    void register_module(const std::string &op_type, Creator creator) { creators[op_type] = creator; }
    Module *create(fbs::FbsModel *fbs_model, const std::string &op_type, const std::string name)
    {
        register_dl_modules();
        auto it = creators.find(op_type);
        if (it == creators.end()) {
            ESP_LOGE("ModuleCreator", "Operation %s is not supported by the B200 backend.", op_type.c_str());
            return nullptr;
        }
        return it->second(fbs_model, name);
    }
    void register_dl_modules(); ///< registers every operator of this backend under the reference's op-type strings
    void clear() { creators.clear(); registered = false; }
    std::vector<std::string> registered_ops()
    {
        register_dl_modules();
        std::vector<std::string> v;
        for (auto &kv : creators) v.push_back(kv.first);
        return v;
    }

private:
    std::map<std::string, Creator> creators;
    bool registered = false;
};

} // namespace module
} // namespace dl
