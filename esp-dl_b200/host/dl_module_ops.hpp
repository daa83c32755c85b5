// Operator modules of the B200 backend.  Each class keeps the name, constructor-argument meaning,
// shape rule and `deserialize` attribute names of the reference module it replaces
// (esp-dl/dl/module/include/dl_module_<op>.hpp); forward() enqueues the CUDA kernel through the C ABI.
#pragma once
#include "dl_module_base.hpp"

namespace dl {
namespace module {

/// Conv (dense or depthwise), reference: dl_module_conv.hpp:17-239.  pads are [top, bottom, left, right].
class Conv : public Module {
public:
    Conv(activation_type_t activation = Linear, std::vector<int> pads = {}, std::vector<int> dilations = {},
         std::vector<int> strides = {}, const char *name = nullptr, const int group = 1, quant_type_t quant_type = QUANT_TYPE_NONE,
         const std::string &target = "c");
    ~Conv();
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    esp_err_t prepare(ModelContext *context) override;
    size_t workspace_bytes(ModelContext *context) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
    void print() override;
    /// Fuse a following 8-bit LUT node (Swish, Sigmoid, ... exported as tables) into the epilogue.  The conv takes
    /// ownership of the table and keeps requantising to `pre_lut_exponent`, the exponent of the tensor that stood
    /// between the two nodes; its output tensor is then the LUT node's.
    void set_fused_lut(TensorBase *table, int pre_lut_exponent)
    {
        m_lut = table;
        m_pre_lut_exponent = pre_lut_exponent;
    }
    /// Fuse a following per-channel activation (PRelu) as one 256-entry table per output channel, `tables` = int8[Cout * 256]
    /// (entry [c][(uint8)q ^ 0x80]); every conv kernel applies such tables in its general epilogue.
    void set_fused_channel_tables(TensorBase *tables, int pre_lut_exponent)
    {
        m_lut = tables;
        m_lut_stride = 256;
        m_pre_lut_exponent = pre_lut_exponent;
    }
    bool can_fuse_channel_tables() const
    {
        return !m_gemm && quant_type == QUANT_TYPE_SYMM_8BIT && !m_lut && !m_residual && (activation == Linear || activation == ReLU);
    }
    /// True for the convs whose kernels apply a table in their staged epilogue: dense int8, no residual, no table yet.
    bool can_fuse_lut() const { return m_group == 1 && quant_type == QUANT_TYPE_SYMM_8BIT && !m_lut && !m_residual && (activation == Linear || activation == ReLU); }
    /// True for a pointwise int8 conv (1x1, stride 1, no padding, group 1) without a fused table: the shapes whose
    /// kernels can add a residual to their result.
    bool can_fold_add() const;
    /// Fold a following Add into the epilogue: the module's LAST input is then the residual tensor.
    void set_residual() { m_residual = true; }
    /// A conv has a bias when it has a third input that is not the residual of a folded Add (a reference Conv may
    /// come without one: dl_module_conv.hpp:137-140).
    bool has_bias() const { return m_inputs_index.size() > (m_residual ? 3u : 2u); }

    /// Geometry the block-fusion pass of dl::Model looks at.
    bool is_depthwise() const { return m_group != 1; }
    bool is_pointwise() const;   ///< stride 1, dilation 1, no padding, group 1, not a Gemm view, no fused table; the
                                 ///< caller checks that the filter is [1,1,Cin,Cout] (filter_is_1x1)
    /// True when the filter tensor's declared shape is [1, 1, Cin, Cout].
    static bool filter_is_1x1(const TensorBase *filter) { return filter && filter->shape.size() == 4 && filter->shape[0] == 1 && filter->shape[1] == 1; }
    bool is_dw3x3() const;       ///< depthwise, stride 1 or 2 (both axes), dilation 1, pads of at most 1
    void skip_pixel_grouping() { m_no_grouping = true; }
    /// Pixels a pointwise int8 conv treats as one row (1 = none) for these channel counts and this many pixels per image.
    static int choose_pixel_group(int cin, int cout, long long pixels);
    /// Channel slices on either side: the int8 kernels that take a pixel stride (not the pixel-grouped pointwise form, the
    /// banded 8/16-channel 3x3 kernel or the 3-channel first layer, which read or write runs of whole pixels).
    bool strided_input_ok(int i, const std::vector<std::vector<int>> &input_shapes) const override { return i == 0 && strided_ok(input_shapes); }
    bool strided_output_ok(int o, const std::vector<std::vector<int>> &input_shapes) const override { return o == 0 && strided_ok(input_shapes); }
    int stride() const { return m_strides[0]; }
    const std::vector<int> &pads() const { return m_pads; }
    friend class FusedBlock;

protected:
    int fill_desc(ModelContext *context, void *desc);
    bool strided_ok(const std::vector<std::vector<int>> &input_shapes) const;
    bool m_no_grouping = false;
    std::vector<int> m_dilations, m_strides;
    const int m_group;
    activation_type_t activation;
    std::vector<int> m_pads;
    std::string m_target;
    bool m_gemm = false;             ///< Gemm / MatMul view: rows = all leading dims
    bool m_residual = false;         ///< the last input is a residual added to the result (a folded Add)
    void *m_dev_exponents = nullptr; ///< int32[out_c] on the device when the filter is per-channel
    // Pixel grouping for pointwise convs whose channel count is not a multiple of 16 (the tensor-core tile kernel
    // needs 16-byte rows): m_group_px consecutive pixels are treated as one pixel with m_group_px * Cin channels,
    // and the filter becomes block diagonal, [g*Cout][g*Cin].  NHWC memory is unchanged on both sides.
    int m_group_px = 1;
    void *m_grp_filter = nullptr, *m_grp_bias = nullptr, *m_grp_exponents = nullptr;
    TensorBase *m_lut = nullptr;     ///< fused 8-bit table (owned)
    int m_lut_stride = 0;            ///< 0: one table; 256: one table per output channel
    int m_pre_lut_exponent = 0;      ///< what the accumulator is requantised to before the table is applied
    bool m_prepared = false;
};

/// An inverted-residual block run as ONE launch of espdl_b200_fused_block: [1x1 expand conv ->] 3x3 depthwise conv ->
/// 1x1 project conv [-> Add].  Built by dl::Model's fusion pass from the Conv modules of the separate nodes (which it
/// owns from then on); the reference runs those nodes one by one (dl_module_conv.hpp, dl_module_add.hpp:43-82).
/// Inputs: x, then the parameters of the convs in their order, then (with a folded Add) the residual tensor.
class FusedBlock : public Module {
public:
    FusedBlock(Conv *expand, Conv *dw, Conv *project, int e_expand, int e_dw, bool residual, const char *name);
    ~FusedBlock();
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    esp_err_t prepare(ModelContext *context) override;

private:
    Conv *m_expand, *m_dw, *m_project;
    int m_e_expand, m_e_dw;
    bool m_residual;
};

/// Gemm (fully connected), reference: dl_module_gemm.hpp:17-168: a 1x1 conv over {1,1,M,K}.
class Gemm : public Conv {
public:
    Gemm(activation_type_t activation = Linear, const char *name = nullptr, quant_type_t quant_type = QUANT_TYPE_NONE,
         const std::string &target = "c");
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
};

/// MatMul of two activations, reference: dl_module_matmul.hpp:16-526.  Shapes of one to four dims with the reference's
/// broadcasting of the leading dims; per-tensor exponents, no bias, optional ReLU.  The reference hands input1 to its
/// conv kernel as the FILTER, and its generic C kernel reads a filter's memory as [N][K] (dl_base_conv2d.cpp:23-32):
/// out[m][n] = act(rnd(sum_k in0[m][k] * in1_flat[n*K + k])).  That reading is reproduced here, so results equal the
/// reference's C path bit for bit (for a mathematically plain product the graph has to store input1 as [N][K]).
class MatMul : public Module {
public:
    MatMul(activation_type_t activation = Linear, const char *name = nullptr, quant_type_t quant_type = QUANT_TYPE_NONE)
        : Module(name, MODULE_NON_INPLACE, quant_type), m_activation(activation) {}
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    esp_err_t prepare(ModelContext *context) override; ///< uploads an operand that is a parameter (a constant weight matrix)
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    size_t workspace_bytes(ModelContext *context) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);

protected:
    activation_type_t m_activation;
    bool slices(ModelContext *context, std::vector<int> &b0, std::vector<int> &b1, int &M, int &K, int &N);
};

/// Add / Sub / Mul with numpy broadcasting, reference: dl_module_add.hpp:14-105, dl_module_mul.hpp, dl_module_sub.hpp.
class Elementwise : public Module {
public:
    Elementwise(int op, const char *name, module_inplace_t inplace, quant_type_t quant_type) : Module(name, inplace, quant_type), m_op(op) {}
    esp_err_t prepare(ModelContext *context) override; ///< uploads an operand that is a parameter (e.g. a scalar factor)
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    /// Channel slices: operands of the output's shape (no broadcast), not Div.
    bool strided_input_ok(int i, const std::vector<std::vector<int>> &input_shapes) const override { return i < 2 && same_shapes(input_shapes); }
    bool strided_output_ok(int o, const std::vector<std::vector<int>> &input_shapes) const override { return o == 0 && same_shapes(input_shapes); }

protected:
    bool same_shapes(const std::vector<std::vector<int>> &input_shapes) const;
    int m_op;
};
class Add : public Elementwise {
public:
    Add(const char *name = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE, quant_type_t quant_type = QUANT_TYPE_NONE);
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
};
class Sub : public Elementwise {
public:
    Sub(const char *name = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE, quant_type_t quant_type = QUANT_TYPE_NONE);
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
};
class Mul : public Elementwise {
public:
    Mul(const char *name = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE, quant_type_t quant_type = QUANT_TYPE_NONE);
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
};
/// Max / Min (dl_module_max.hpp, dl_module_min.hpp), Div (dl_module_div.hpp), Mod (dl_module_mod.hpp, fmod form) and the
/// comparisons with a bool output (dl_module_greater.hpp, dl_module_greater_or_equal.hpp, dl_module_equal.hpp,
/// dl_module_less.hpp, dl_module_less_or_equal.hpp): same broadcasting and construction as Add.
#define ESPDL_B200_TWO_OPERAND_MODULE(NAME)                                                                                        \
    class NAME : public Elementwise {                                                                                              \
    public:                                                                                                                        \
        NAME(const char *name = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE, quant_type_t quant_type = QUANT_TYPE_NONE); \
        static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);                                               \
    };
ESPDL_B200_TWO_OPERAND_MODULE(Max)
ESPDL_B200_TWO_OPERAND_MODULE(Min)
ESPDL_B200_TWO_OPERAND_MODULE(Div)
ESPDL_B200_TWO_OPERAND_MODULE(Mod)
ESPDL_B200_TWO_OPERAND_MODULE(Greater)
ESPDL_B200_TWO_OPERAND_MODULE(GreaterOrEqual)
ESPDL_B200_TWO_OPERAND_MODULE(Equal)
ESPDL_B200_TWO_OPERAND_MODULE(Less)
ESPDL_B200_TWO_OPERAND_MODULE(LessOrEqual)
#undef ESPDL_B200_TWO_OPERAND_MODULE

/// Pow (reference: dl_module_pow.hpp:17-110, dl_base_pow.cpp:9-63): round(powf(a * 2^ea, b * 2^eb) * 2^-eo) with numpy
/// broadcasting.  For int8 the 256 x 256 possible answers are computed once on the host with its own powf and the kernel
/// looks them up, which makes the result the reference's bit for bit; int16 calls powf on the device.
class Pow : public Elementwise {
public:
    Pow(const char *name = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE, quant_type_t quant_type = QUANT_TYPE_NONE);
    ~Pow();
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);

protected:
    void *m_dev_table = nullptr;
    int m_table_key[4] = {0x7fffffff, 0, 0, 0}; ///< exponents and rounding mode the table was built for
};

/// One-input elementwise modules: RequantizeLinear / QuantizeLinear / DequantizeLinear
/// (dl_module_requantize_linear.hpp:8-60), LUT and every activation exported with a `lut` attribute
/// (dl_module_lut.hpp:15-104), Clip (dl_module_clip.hpp), Relu (dl_module_relu.hpp), PRelu (dl_module_prelu.hpp).
class Unary : public Module {
public:
    Unary(int op, const char *name, module_inplace_t inplace, quant_type_t quant_type, TensorBase *param = nullptr) :
        Module(name, inplace, quant_type), m_op(op), m_param(param)
    {
    }
    ~Unary() { delete m_param; }
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override { return {input_shapes[0]}; }
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    esp_err_t prepare(ModelContext *context) override;
    TensorBase *get_table() { return m_param; }
    /// Hands the table (or PReLU slopes) to the caller, who owns it from then on.
    TensorBase *release_table()
    {
        TensorBase *t = m_param;
        m_param = nullptr;
        return t;
    }
    int op() const { return m_op; }
    /// Channel slices: every one-operand operator but PRelu (its slopes broadcast over the leading axes).
    bool strided_input_ok(int i, const std::vector<std::vector<int>> &input_shapes) const override;
    bool strided_output_ok(int o, const std::vector<std::vector<int>> &input_shapes) const override { return strided_input_ok(o, input_shapes); }

protected:
    int m_op;
    TensorBase *m_param; ///< LUT table or PReLU alpha (owned)
    int m_clip_lo = -128, m_clip_hi = 127;
};
class RequantizeLinear : public Unary {
public:
    RequantizeLinear(const char *name = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE, quant_type_t quant_type = QUANT_TYPE_NONE);
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
};
class LUT : public Unary {
public:
    LUT(const char *name = nullptr, TensorBase *table = nullptr, module_inplace_t inplace = MODULE_INPLACE_CHANGED_BUFFER,
        quant_type_t quant_type = QUANT_TYPE_NONE);
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
};
class Clip : public Unary {
public:
    Clip(const char *name = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE, quant_type_t quant_type = QUANT_TYPE_NONE);
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
};
class Relu : public Unary {
public:
    Relu(const char *name = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE, quant_type_t quant_type = QUANT_TYPE_NONE);
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
};
class PRelu : public Unary {
public:
    PRelu(const char *name = nullptr, TensorBase *alpha = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE,
          quant_type_t quant_type = QUANT_TYPE_NONE);
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
};

/// MaxPool / AveragePool / GlobalAveragePool, reference: dl_module_max_pool.hpp, dl_module_average_pool.hpp,
/// dl_module_global_average_pool.hpp.  Unlike the reference, GlobalAveragePool keeps the batch extent.
class Pool : public Module {
public:
    Pool(int op, const char *name, const std::vector<int> &kernel, const std::vector<int> &pads, const std::vector<int> &strides,
         quant_type_t quant_type) :
        Module(name, MODULE_NON_INPLACE, quant_type), m_op(op), m_kernel(kernel), m_pads(pads), m_strides(strides)
    {
    }
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;

protected:
    int m_op;
    std::vector<int> m_kernel, m_pads, m_strides;
};
class MaxPool : public Pool {
public:
    MaxPool(const char *name = nullptr, const std::vector<int> &filter_shape = {2, 2}, const std::vector<int> &padding = {},
            const std::vector<int> &strides = {1, 1}, quant_type_t quant_type = QUANT_TYPE_NONE);
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
};
class AveragePool : public Pool {
public:
    AveragePool(const char *name = nullptr, const std::vector<int> &kernel_shape = {2, 2}, const std::vector<int> &pads = {},
                const std::vector<int> &strides = {1, 1}, quant_type_t quant_type = QUANT_TYPE_NONE);
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
};
class GlobalAveragePool : public Pool {
public:
    GlobalAveragePool(const char *name = nullptr, quant_type_t quant_type = QUANT_TYPE_NONE);
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
};

/// Resize (nearest), reference: dl_module_resize.hpp.
class Resize : public Module {
public:
    Resize(const char *name = nullptr, const resize_mode_t resize_mode = RESIZE_NEAREST, const std::vector<float> scales = {},
           const std::vector<int64_t> sizes = {}, const bool align_corners = false, quant_type_t quant_type = QUANT_TYPE_NONE);
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
    bool strided_output_ok(int o, const std::vector<std::vector<int>> &input_shapes) const override
    {
        return o == 0 && quant_type == QUANT_TYPE_SYMM_8BIT && !input_shapes.empty() && input_shapes[0].size() >= 3;
    }

protected:
    resize_mode_t m_resize_mode;
    std::vector<float> m_scales;
    std::vector<int64_t> m_sizes;
    bool m_align_corners;
};

/// Concat (dl_module_concat.hpp), Split (dl_module_split.hpp), Transpose (dl_module_transpose.hpp): strided copies.
class Concat : public Module {
public:
    Concat(const char *name = nullptr, int axis = 0, quant_type_t quant_type = QUANT_TYPE_NONE) :
        Module(name, MODULE_NON_INPLACE, quant_type), axis(axis)
    {
    }
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
    int get_axis() const { return axis; }
    /// A part may be a channel slice when the parts move as 16-byte units in one launch (last axis, whole units).
    bool strided_input_ok(int i, const std::vector<std::vector<int>> &input_shapes) const override;

protected:
    int axis;
};
class Split : public Module {
public:
    Split(TensorBase *split = nullptr, int axis = 0, int num_outputs = -1, const char *name = nullptr,
          module_inplace_t inplace = MODULE_NON_INPLACE, quant_type_t quant_type = QUANT_TYPE_NONE);
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
    int get_axis() const { return m_axis; }
    bool strided_output_ok(int o, const std::vector<std::vector<int>> &input_shapes) const override;

protected:
    std::vector<int> m_split;
    int m_axis, m_num_outputs;
};
/// ReduceMean / ReduceSum / ReduceMax / ReduceMin (reference: dl_module_reduce_base.hpp:15-262 and the modules built on it).
class Reduce : public Module {
public:
    Reduce(int op, int keepdims, std::vector<bool> axes_reduce_flag, const char *name = nullptr, quant_type_t quant_type = QUANT_TYPE_NONE) :
        Module(name, MODULE_NON_INPLACE, quant_type), m_op(op), m_keepdims(keepdims), m_axes_reduce_flag(axes_reduce_flag)
    {
    }
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);

    ~Reduce();

protected:
    int m_op, m_keepdims;
    std::vector<bool> m_axes_reduce_flag;
    void *m_dev_table = nullptr; ///< ReduceLogSumExp on int8: the exp table (tool::gen_lut_8bit(expf)) on the device
    int m_table_exponent = 0x7fffffff;
};

/// Slice with positive steps (reference: dl_module_slice.hpp:10-128, TensorBase::slice); a strided device copy.
class Slice : public Module {
public:
    Slice(std::vector<int> start, std::vector<int> end, std::vector<int> axes = {}, std::vector<int> step = {}, const char *name = nullptr,
          quant_type_t quant_type = QUANT_TYPE_NONE) :
        Module(name, MODULE_NON_INPLACE, quant_type), m_start(start), m_end(end), m_axes(axes), m_step(step)
    {
    }
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);

protected:
    /// per input axis: first index, count, step (after the reference's normalisation of negative and oversized bounds)
    bool resolve(const std::vector<int> &shape, std::vector<int> &first, std::vector<int> &count, std::vector<int> &step) const;
    std::vector<int> m_start, m_end, m_axes, m_step;
};

/// Pad (reference: dl_module_pad.hpp:10-100): constant / edge / reflect, pads = [begin per axis ..., end per axis ...].
class Pad : public Module {
public:
    Pad(std::vector<int> pads, int mode, long long constant, const char *name = nullptr, quant_type_t quant_type = QUANT_TYPE_NONE) :
        Module(name, MODULE_NON_INPLACE, quant_type), m_pads(pads), m_mode(mode), m_constant(constant)
    {
    }
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);

protected:
    std::vector<int> m_pads;
    int m_mode;
    long long m_constant;
};

class Transpose : public Module {
public:
    Transpose(const char *name = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE, quant_type_t quant_type = QUANT_TYPE_NONE,
              std::vector<int> perm = {}) :
        Module(name, inplace, quant_type), m_perm(perm)
    {
    }
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);

protected:
    std::vector<int> m_perm;
};

/// SpaceToDepth (dl_module_space_to_depth.hpp) and DepthToSpace "DCR" / "CRD" (dl_module_depth_to_space.hpp) of an NHWC
/// tensor: one launch of the strided-copy kernel over a six-axis view.  The reference's DCR index rule addresses the output
/// consistently only when the output has `blocksize` channels; any other DCR shape fails with ESPDL_ERR_UNSUPPORTED.
class SpaceToDepth : public Module {
public:
    SpaceToDepth(int blocksize = 2, const char *name = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE,
                 quant_type_t quant_type = QUANT_TYPE_NONE) :
        Module(name, inplace, quant_type), m_blocksize(blocksize)
    {
    }
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);

protected:
    int m_blocksize;
};
class DepthToSpace : public Module {
public:
    DepthToSpace(int blocksize = 2, std::string mode = "DCR", const char *name = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE,
                 quant_type_t quant_type = QUANT_TYPE_NONE) :
        Module(name, inplace, quant_type), m_blocksize(blocksize), m_mode(mode)
    {
    }
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);

protected:
    int m_blocksize;
    std::string m_mode;
};

/// InsertZeros (dl_module_insert_zeros.hpp; the first half of a transposed convolution): the output is cleared and the
/// input pixels are scattered `stride` apart along the one or two spatial axes of an NWC / NHWC tensor.
class InsertZeros : public Module {
public:
    InsertZeros(const char *name = nullptr, const std::vector<int> &stride = {1}, const std::vector<int> &output_padding = {0},
                quant_type_t quant_type = QUANT_TYPE_NONE) :
        Module(name, MODULE_NON_INPLACE, quant_type), m_stride(stride), m_output_padding(output_padding)
    {
    }
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);

protected:
    std::vector<int> m_stride, m_output_padding;
};

/// StreamingCache (dl_module_streaming_cache.hpp): keeps the last `window_size - 1` frames of its input between runs and puts
/// them in front of the new frames: output = [cache | input], then cache = the output's last cache-size bytes (byte
/// ranges of the flat tensors, as the reference copies them).  The cache lives in device memory and starts as zeros;
/// reset() clears it.
class StreamingCache : public Module {
public:
    StreamingCache(const char *name = nullptr, int window_size = 1, int frame_axis = 1, module_inplace_t inplace = MODULE_NON_INPLACE,
                   quant_type_t quant_type = QUANT_TYPE_NONE) :
        Module(name, inplace, quant_type), m_window_size(window_size), m_frame_axis(frame_axis), m_cache(nullptr), m_cache_bytes(0)
    {
    }
    ~StreamingCache();
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    esp_err_t prepare(ModelContext *context) override;
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    void reset() override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);

protected:
    int m_window_size, m_frame_axis;
    void *m_cache;
    size_t m_cache_bytes;
};

/// Gather along one axis with constant indices (dl_module_gather.hpp): the module owns `indices` (int32 or int64, any
/// shape); prepare() checks them against the axis length and uploads them as int32.
class Gather : public Module {
public:
    Gather(TensorBase *indices, int axis = 0, const char *name = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE,
           quant_type_t quant_type = QUANT_TYPE_NONE) :
        Module(name, inplace, quant_type), m_indices(indices), m_axis(axis), m_dev_indices(nullptr)
    {
    }
    ~Gather();
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    esp_err_t prepare(ModelContext *context) override;
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);

protected:
    TensorBase *m_indices;
    int m_axis;
    TensorBase *m_dev_indices; ///< the indices as int32 with a device copy
};

/// RMSNormalization (dl_module_rms_normalization.hpp; inputs x and a float scale) and LayerNormalization
/// (dl_module_layer_normalization.hpp; inputs x [, scale [, bias]], outputs y [, mean, inv_std_dev]) over the axes from
/// `axis` to the last one.
class Normalization : public Module {
public:
    Normalization(int op, int axis, float epsilon, const char *name, module_inplace_t inplace, quant_type_t quant_type) :
        Module(name, inplace, quant_type), m_op(op), m_axis(axis), m_epsilon(epsilon)
    {
    }
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    esp_err_t prepare(ModelContext *context) override; ///< uploads scale / bias when they are parameters
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;

protected:
    int m_op, m_axis;
    float m_epsilon;
};
class RMSNormalization : public Normalization {
public:
    RMSNormalization(int axis = -1, float epsilon = 1e-5f, const char *name = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE,
                     quant_type_t quant_type = QUANT_TYPE_NONE);
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
};
class LayerNormalization : public Normalization {
public:
    LayerNormalization(int axis = -1, float epsilon = 1e-5f, int stash_type = 1, const char *name = nullptr,
                       module_inplace_t inplace = MODULE_NON_INPLACE, quant_type_t quant_type = QUANT_TYPE_NONE);
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
};

/// Reshape / Flatten / Squeeze / Unsqueeze / Identity: the output aliases the input buffer
/// (MODULE_INPLACE_UNCHANGED_BUFFER); forward() is a no-op unless the planner gave it a separate buffer.
class Reshape : public Module {
public:
    enum Kind { RESHAPE, FLATTEN, SQUEEZE, UNSQUEEZE, IDENTITY };
    Reshape(Kind kind, std::vector<int> arg, int axis, const char *name, quant_type_t quant_type) :
        Module(name, MODULE_INPLACE_UNCHANGED_BUFFER, quant_type), m_kind(kind), m_arg(arg), m_axis(axis)
    {
    }
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    static Module *deserialize_reshape(fbs::FbsModel *fbs_model, std::string node_name);
    static Module *deserialize_flatten(fbs::FbsModel *fbs_model, std::string node_name);
    static Module *deserialize_squeeze(fbs::FbsModel *fbs_model, std::string node_name);
    static Module *deserialize_unsqueeze(fbs::FbsModel *fbs_model, std::string node_name);
    static Module *deserialize_identity(fbs::FbsModel *fbs_model, std::string node_name);

protected:
    Kind m_kind;
    std::vector<int> m_arg;
    int m_axis;
};

/// Softmax on int8 input with a host-built exp table, float output (dl_module_softmax.hpp:14-246).
class Softmax : public Module {
public:
    Softmax(const char *name = nullptr, int axis = -1, module_inplace_t inplace = MODULE_NON_INPLACE,
            quant_type_t quant_type = QUANT_TYPE_NONE) :
        Module(name, inplace, quant_type), axis(axis)
    {
    }
    ~Softmax();
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override { return {input_shapes[0]}; }
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);

protected:
    int axis;
    bool m_log = false; ///< LogSoftmax
    void *m_dev_table = nullptr;
    int m_table_exponent = 0x7fffffff;
};

/// LogSoftmax on int8 (reference: dl_module_log_softmax.hpp:150-215): the same exp table and sequential sum as Softmax,
/// y = 2^e_in * x - logf(sum); float output, or int8 / int16 when the following QuantizeLinear is folded in.
class LogSoftmax : public Softmax {
public:
    LogSoftmax(const char *name = nullptr, int axis = -1, module_inplace_t inplace = MODULE_NON_INPLACE, quant_type_t quant_type = QUANT_TYPE_NONE) :
        Softmax(name, axis, inplace, quant_type)
    {
        m_log = true;
    }
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
};

/// LpNormalization along one axis, p = 1 or 2 (reference: dl_module_lp_normalization.hpp:20-360).
class LpNormalization : public Module {
public:
    LpNormalization(int axis = -1, int p = 2, const char *name = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE,
                    quant_type_t quant_type = QUANT_TYPE_NONE) :
        Module(name, inplace, quant_type), m_axis(axis), m_p(p)
    {
    }
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override { return {input_shapes[0]}; }
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);

protected:
    int m_axis, m_p;
};

/// ReverseSequence (reference: dl_module_reverse_sequence.hpp:10-126): inputs x and sequence_lens (int64); batch and time are
/// the first two axes in either order.
class ReverseSequence : public Module {
public:
    ReverseSequence(int batch_axis = 1, int time_axis = 0, const char *name = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE,
                    quant_type_t quant_type = QUANT_TYPE_NONE) :
        Module(name, inplace, quant_type), m_batch_axis(batch_axis), m_time_axis(time_axis)
    {
    }
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override { return {input_shapes[0]}; }
    esp_err_t prepare(ModelContext *context) override; ///< uploads sequence_lens when it is a parameter
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);

protected:
    int m_batch_axis, m_time_axis;
};

/// GRU / LSTM, quantized, batch 1 (reference: dl_module_gru.hpp:12-449, dl_module_lstm.hpp:12-522): inputs X, W, R [, B,
/// sequence_lens, initial_h [, initial_c]], outputs Y, Y_h [, Y_c].  The whole sequence is one kernel launch; the sigmoid and
/// tanh tables (math::SigmoidLUT(-6.3, 6.3), math::TanhLUT(-3.5, 3.5) at gate_exponent) are built on the host.
class Rnn : public Module {
public:
    Rnn(int op, const char *name, int hidden_size, int direction_num, int layout, int gate_exponent, module_inplace_t inplace,
        quant_type_t quant_type) :
        Module(name, inplace, quant_type), m_op(op), m_hidden_size(hidden_size), m_direction_num(direction_num), m_layout(layout),
        m_gate_exponent(gate_exponent)
    {
    }
    ~Rnn();
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override;
    esp_err_t prepare(ModelContext *context) override; ///< uploads W, R, B and the two tables
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;

protected:
    int m_op, m_hidden_size, m_direction_num, m_layout, m_gate_exponent;
    void *m_dev_sigmoid = nullptr, *m_dev_tanh = nullptr;
    int m_sigmoid_max = 0, m_tanh_max = 0;
};
class GRU : public Rnn {
public:
    GRU(const char *name = nullptr, int hidden_size = 0, int direction_num = 1, int layout = 0, int gate_exponent = -8,
        module_inplace_t inplace = MODULE_NON_INPLACE, quant_type_t quant_type = QUANT_TYPE_NONE) :
        Rnn(0, name, hidden_size, direction_num, layout, gate_exponent, inplace, quant_type)
    {
    }
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
};
class LSTM : public Rnn {
public:
    LSTM(const char *name = nullptr, int hidden_size = 0, int direction_num = 1, int layout = 0, int gate_exponent = -8,
         module_inplace_t inplace = MODULE_NON_INPLACE, quant_type_t quant_type = QUANT_TYPE_NONE) :
        Rnn(1, name, hidden_size, direction_num, layout, gate_exponent, inplace, quant_type)
    {
    }
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);
};

/// ScatterND (reference: dl_module_scatter_nd.hpp:20-264): inputs data, indices (int64), updates; reduction none / add / mul /
/// max / min applied slice by slice in the order of the index tuples.
class ScatterND : public Module {
public:
    ScatterND(const std::string &reduction = "none", const char *name = nullptr, module_inplace_t inplace = MODULE_NON_INPLACE,
              quant_type_t quant_type = QUANT_TYPE_NONE);
    std::vector<std::vector<int>> get_output_shape(std::vector<std::vector<int>> &input_shapes) override { return {input_shapes[0]}; }
    esp_err_t prepare(ModelContext *context) override; ///< uploads indices / updates when they are parameters
    void forward(ModelContext *context, runtime_mode_t mode = RUNTIME_MODE_AUTO) override;
    static Module *deserialize(fbs::FbsModel *fbs_model, std::string node_name);

protected:
    int m_reduction;
};

} // namespace module
} // namespace dl
