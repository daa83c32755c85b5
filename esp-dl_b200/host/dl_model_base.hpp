// dl::Model for the B200 backend: load(.espdl) -> topological plan -> device arena planned from tensor
// lifetimes -> run() = one pass of every module's forward() on a CUDA stream (captured once into a CUDA
// graph and replayed).  Public surface follows the reference (esp-dl/dl/model/include/dl_model_base.hpp:46-449).
//
// Differences that come from running on a GPU:
//  * graph inputs / outputs have a pinned HOST buffer (`TensorBase::data`, what users read and write, as with
//    the reference) and a DEVICE buffer; run() copies inputs up and outputs down around the plan;
//  * `input_shapes` may give any batch extent N; every module honours dim 0 (the reference's kernels read
//    one image);
//  * `max_internal_size` is accepted and ignored (one arena in HBM).
#pragma once
#include "dl_module_base.hpp"

#include <map>
#include <string>
#include <vector>

namespace dl {

typedef enum { MEMORY_MANAGER_GREEDY = 0, LINEAR_MEMORY_MANAGER = 1 } memory_manager_t;

/// One planned tensor: where it lives in the arena and for which plan steps it must stay intact.
struct TensorInfo {
    std::string name;
    std::vector<int> shape;
    dtype_t dtype = DATA_TYPE_INT8;
    int exponent = 0;
    int first = 0;          ///< producing step (-1: graph input)
    int last = 0;           ///< last consuming step (INT_MAX: graph output)
    size_t bytes = 0;
    size_t offset = 0;
    int alias_of = -1;      ///< index of the tensor whose buffer this one shares (in-place / view), or -1
    size_t view_offset = 0; ///< bytes from the start of `alias_of`'s buffer (a channel slice of a Concat output / Split input)
    int row_stride = 0;     ///< elements between rows of the last axis when this tensor is such a slice, else 0
    bool is_graph_io = false;
};

/// Lifetime-based arena planner (role of esp-dl/dl/model/src/dl_memory_manager_greedy.cpp:77-427):
/// tensors whose lifetimes do not overlap share memory; best-fit over a free list, 256-byte alignment.
class MemoryManagerGreedy {
public:
    /// Assigns `offset` for every non-aliased tensor; returns the arena size in bytes.
    static size_t plan(std::vector<TensorInfo> &tensors, bool reuse = true);
};

struct module_info {
    std::string type;
    float latency_us = 0;
};

class Model {
public:
    Model() {}
    Model(const char *rodata_address_or_partition_label_or_path, fbs::model_location_type_t location = fbs::MODEL_LOCATION_IN_FLASH_RODATA,
          int max_internal_size = 0, memory_manager_t mm_type = MEMORY_MANAGER_GREEDY, const uint8_t *key = nullptr, bool param_copy = true,
          const std::map<std::string, std::vector<int>> &input_shapes = {});
    Model(const char *rodata_address_or_partition_label_or_path, int model_index,
          fbs::model_location_type_t location = fbs::MODEL_LOCATION_IN_FLASH_RODATA, int max_internal_size = 0,
          memory_manager_t mm_type = MEMORY_MANAGER_GREEDY, const uint8_t *key = nullptr, bool param_copy = true,
          const std::map<std::string, std::vector<int>> &input_shapes = {});
    Model(fbs::FbsModel *fbs_model, int internal_size = 0, memory_manager_t mm_type = MEMORY_MANAGER_GREEDY,
          const std::map<std::string, std::vector<int>> &input_shapes = {});
    virtual ~Model();

    virtual esp_err_t load(const char *rodata_address_or_partition_label_or_path,
                           fbs::model_location_type_t location = fbs::MODEL_LOCATION_IN_FLASH_RODATA, int model_index = 0,
                           const uint8_t *key = nullptr, bool param_copy = true);
    virtual esp_err_t load(fbs::FbsModel *fbs_model);
    virtual void build(size_t max_internal_size, memory_manager_t mm_type = MEMORY_MANAGER_GREEDY, bool preload = false,
                       const std::map<std::string, std::vector<int>> &input_shapes = {});

    /// Upload the graph inputs' host buffers, execute the plan, download the graph outputs, synchronise.
    virtual void run(runtime_mode_t mode = RUNTIME_MODE_SINGLE_CORE);
    virtual void run(TensorBase *input, runtime_mode_t mode = RUNTIME_MODE_SINGLE_CORE);
    virtual void run(std::map<std::string, TensorBase *> &user_inputs, runtime_mode_t mode = RUNTIME_MODE_SINGLE_CORE,
                     std::map<std::string, TensorBase *> user_outputs = {});
    /// Time slice of the plan, as the reference's staged run (dl_model_base.cpp:240-260).
    virtual void run(int stage_num, int stage_index, runtime_mode_t mode = RUNTIME_MODE_SINGLE_CORE);
    /// Execute the plan on the device-resident inputs only (no host copies); asynchronous unless `sync`.
    esp_err_t run_device(bool sync = true);
    /// Pipelined form of run() for a stream of batches.  submit() uploads the inputs' host buffers (it returns once
    /// that copy is done, so the buffers may be refilled at once), then enqueues the plan and the download of the
    /// outputs without waiting for them; the upload of one submission overlaps the execution of the one before it
    /// (second stream, a staging buffer per input).  wait() blocks until the OLDEST outstanding submission has
    /// finished and copies its outputs into the outputs' host buffers.  At most two submissions may be outstanding.
    esp_err_t submit();
    esp_err_t wait();

    esp_err_t test();
    std::map<std::string, module_info> get_module_info();
    void profile_module(bool sort_module_by_latency = false);
    void profile_memory();
    void profile(bool sort_module_by_latency = false);

    virtual std::map<std::string, TensorBase *> &get_inputs() { return m_inputs; }
    virtual TensorBase *get_input() { return m_inputs.empty() ? nullptr : m_inputs.begin()->second; }
    virtual TensorBase *get_input(const std::string &name);
    virtual TensorBase *get_intermediate(const std::string &name);
    virtual std::map<std::string, TensorBase *> &get_outputs() { return m_outputs; }
    virtual TensorBase *get_output() { return m_outputs.empty() ? nullptr : m_outputs.begin()->second; }
    virtual TensorBase *get_output(const std::string &name);
    std::string get_metadata_prop(const std::string &key);
    virtual void print();
    virtual void reset();
    /// Releases what inference does not need (reference: dl_model_base.cpp:431-440): the host copies of parameters that
    /// are resident on the device (filters, biases, tables; small operands that modules read on the host are kept), the
    /// FlatBuffers name maps and the module registry.  Model::test() and graph inspection no longer work afterwards.
    void minimize();
    virtual fbs::FbsModel *get_fbs_model() { return m_fbs_model; }

    // backend knobs (set before build / the constructor reads the environment for defaults)
    bool m_use_graph = true;     ///< replay the plan as a captured CUDA graph
    int m_slice_views = 0;       ///< tensors placed as channel slices of a Concat output / Split input (no copy)
    bool m_plan_only = false;    ///< build() stops after the arena plan: no device is touched (planner tests on CPU)
    const std::vector<TensorInfo> &tensor_infos() const { return m_tensor_infos; }
    bool m_reuse_memory = true;  ///< false: every tensor keeps its own buffer (lets tests read intermediates)
    int m_status = 0;            ///< first failing C-ABI status, 0 if none
    size_t arena_bytes() const { return m_arena_bytes; }
    size_t num_modules() const { return m_execution_plan.size(); }
    /// Tensors that live as channel slices inside a Concat output / Split input (ESPDL_B200_SLICE_VIEWS=0 switches them off).
    int num_slice_views() const { return m_slice_views; }
    void *stream() { return m_model_context ? m_model_context->stream : nullptr; }
    int round_mode() const { return m_model_context ? (int)m_model_context->round_mode : 0; }

protected:
    esp_err_t execute(int first, int last);
    void release();
    fbs::FbsLoader *m_fbs_loader = nullptr;
    fbs::FbsModel *m_fbs_model = nullptr;
    bool m_own_fbs_model = false;
    std::vector<module::Module *> m_execution_plan;
    std::vector<std::string> m_module_types;
    std::vector<std::vector<std::string>> m_module_inputs, m_module_outputs;
    ModelContext *m_model_context = nullptr;
    std::map<std::string, TensorBase *> m_inputs, m_outputs;
    std::string m_name, m_doc_string;
    int64_t m_version = 0;
    void *m_arena = nullptr;
    size_t m_arena_bytes = 0;
    void *m_graph = nullptr;
    // Pipelined passes (submit / wait) run the plan in two parts: the steps that read a graph input, then the rest.  Once the
    // first part of a pass is done its input buffers are free again, so the next pass's upload goes straight into them while
    // the second part runs - no staging copy.  m_input_steps = number of leading steps that belong to the first part.
    void *m_graph_head = nullptr, *m_graph_tail = nullptr;
    int m_input_steps = 0;
    esp_err_t run_part(bool head);
    // submit()/wait() state
    void *m_copy_stream = nullptr, *m_ev_uploaded = nullptr, *m_ev_consumed = nullptr, *m_ev_done[2] = {nullptr, nullptr};
    std::map<std::string, void *> m_in_stage;                 ///< device staging buffer per graph input
    std::map<std::string, void *> m_out_stage[2];             ///< pinned host staging per graph output, two slots
    long long m_submitted = 0, m_collected = 0;
    void release_pipeline();
    void fold_residual_adds();
    int alias_channel_slices(std::vector<TensorInfo> &infos, std::map<std::string, int> &info_index,
                             const std::vector<std::vector<std::vector<int>>> &step_in_shapes, std::vector<bool> &is_root);
    void fold_luts();
    /// A PRelu that is the only reader of an int8 conv's output becomes that conv's per-channel tables (one launch less; the
    /// conv's kernels apply them in their general epilogue).  ESPDL_B200_FOLD_PRELU=0 switches the pass off.
    void fold_prelus();
    /// A QuantizeLinear whose only input is the float output of a Softmax / LogSoftmax with no other reader disappears: the softmax
    /// kernel writes the quantized tensor itself (the same `round(y * 2^-e)` on the same float).  ESPDL_B200_FOLD_QUANT=0 keeps it.
    void fold_quantize_after_softmax();
    void fuse_blocks();
    bool m_built = false;
    std::vector<TensorInfo> m_tensor_infos;
};

} // namespace dl
