// C binding of the Arm NN runtime API for hosts that are not C++ (the Python tests and bench.py of this repository):
// INetwork -> Optimize(backend list) -> IRuntime::LoadNetwork -> EnqueueWorkload, for any registered backend id
// ("B200Acc" loaded as a dynamic backend from armnn_b200/backend/, or "CpuRef").  It wraps the UNMODIFIED Arm NN
// runtime (libarmnn.so) and adds no computation of its own: every call below is one or two calls of
// include/armnn/INetwork.hpp / IRuntime.hpp of the Arm NN tree.
//
//   build: python -m armnn_b200.build   (needs $ARMNN_ROOT for the headers and a libarmnn.so to link against)
#include <armnn/ArmNN.hpp>
#include <armnn/BackendRegistry.hpp>

#include <algorithm>
#include <sstream>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "../../include/b200k.h"

using namespace armnn;

static thread_local std::string g_err;
extern "C" const char* armnnc_last_error() { return g_err.c_str(); }

namespace {

DataType act_type(int dt)
{
    switch (dt) {
        case B200K_U8:  return DataType::QAsymmU8;
        case B200K_S8:  return DataType::QAsymmS8;
        case B200K_S16: return DataType::QSymmS16;
        case B200K_S32: return DataType::Signed32;
        case 5:         return DataType::Boolean;         // bridge only: the kernels see a Boolean tensor as bytes
        case 6:         return DataType::Float16;         // bridge only: the operand of the two fp16 conversion layers
        default:        return DataType::Float32;
    }
}

// TensorInfo of an operand; per-axis scales (weights / bias) when t.scales != NULL.
TensorInfo make_info(const b200k_qtensor& t, const TensorShape& shape, unsigned axis_dim, unsigned n_axis,
                     bool constant)
{
    TensorInfo info(shape, act_type(t.dtype));
    if (t.scales) {
        if (t.dtype == B200K_S8) info.SetDataType(DataType::QSymmS8);
        info.SetQuantizationScales(std::vector<float>(t.scales, t.scales + n_axis));
        info.SetQuantizationDim(Optional<unsigned int>(axis_dim));
    } else if (t.dtype != B200K_F32 && t.dtype != 5 && t.dtype != 6) {
        info.SetQuantizationScale(t.scale);
        info.SetQuantizationOffset(t.zero_point);
    }
    info.SetConstant(constant);
    return info;
}

}  // namespace


namespace {

struct CNet {
    INetworkPtr net{nullptr, nullptr};
    std::vector<IConnectableLayer*> layers;              // index = handle returned to the caller
    std::vector<std::vector<uint8_t>> blobs;             // constant data kept alive until Optimize
    std::vector<std::pair<int, TensorInfo>> inputs, outputs;   // binding id, info
};

struct CRuntime {
    IRuntimePtr rt{nullptr, nullptr};
};

struct CLoaded {
    CRuntime* rt;
    NetworkId id;
    std::vector<std::pair<int, TensorInfo>> inputs, outputs;
    // IRuntime::ImportInputs / ImportOutputs state of armnnc_enqueue_preimported
    std::vector<const void*> pre_in_ptrs;
    std::vector<void*> pre_out_ptrs;
    std::vector<ImportedInputId> pre_in;
    std::vector<ImportedOutputId> pre_out;
};

TensorInfo info_from(int dtype, int rank, const int32_t* shape, float scale, int32_t zp, const float* scales,
                     int n_scales, int axis, bool constant)
{
    unsigned dims[5];
    for (int i = 0; i < rank; ++i) dims[i] = (unsigned)shape[i];
    b200k_qtensor t{nullptr, dtype, scale, zp, scales};
    return make_info(t, TensorShape((unsigned)rank, dims), (unsigned)axis, (unsigned)n_scales, constant);
}

}  // namespace

extern "C" {

void* armnnc_runtime_create(const char* dynamic_backend_path)
{
    try {
        IRuntime::CreationOptions opts;
        if (dynamic_backend_path && *dynamic_backend_path) opts.m_DynamicBackendsPath = dynamic_backend_path;
        auto* r = new CRuntime;
        r->rt = IRuntime::Create(opts);
        return r;
    } catch (const std::exception& e) { g_err = e.what(); return nullptr; }
}
// The same with BackendOptions("B200Acc", {...}) for the runtime: device_id >= 0 sets "DeviceId", graph_replay 0 / 1
// sets "GraphReplay" (-1: leave the default), selftest_us > 0 sets "WaitSelfTestUs".
void* armnnc_runtime_create_ex(const char* dynamic_backend_path, int device_id, int graph_replay, int selftest_us)
{
    try {
        IRuntime::CreationOptions opts;
        if (dynamic_backend_path && *dynamic_backend_path) opts.m_DynamicBackendsPath = dynamic_backend_path;
        BackendOptions bo("B200Acc");
        if (device_id >= 0) bo.AddOption(BackendOptions::BackendOption("DeviceId", device_id));
        if (graph_replay >= 0) bo.AddOption(BackendOptions::BackendOption("GraphReplay", graph_replay != 0));
        if (selftest_us > 0) bo.AddOption(BackendOptions::BackendOption("WaitSelfTestUs", selftest_us));
        opts.m_BackendOptions.push_back(bo);
        auto* r = new CRuntime;
        r->rt = IRuntime::Create(opts);
        return r;
    } catch (const std::exception& e) { g_err = e.what(); return nullptr; }
}
void armnnc_runtime_destroy(void* r) { delete static_cast<CRuntime*>(r); }

// 1 when `id` is a registered backend of this runtime
int armnnc_backend_available(void* r, const char* id)
{
    (void)r;
    return BackendRegistryInstance().IsBackendRegistered(BackendId(id)) ? 1 : 0;
}

void* armnnc_network_create()
{
    auto* n = new CNet;
    n->net = INetwork::Create();
    return n;
}
void armnnc_network_destroy(void* n) { delete static_cast<CNet*>(n); }

static int add_layer(CNet* n, IConnectableLayer* l) { n->layers.push_back(l); return (int)n->layers.size() - 1; }

int armnnc_add_input(void* vn, int binding, int dtype, int rank, const int32_t* shape, float scale, int32_t zp)
{
    auto* n = static_cast<CNet*>(vn);
    auto* l = n->net->AddInputLayer(binding);
    TensorInfo info = info_from(dtype, rank, shape, scale, zp, nullptr, 0, 0, false);
    l->GetOutputSlot(0).SetTensorInfo(info);
    n->inputs.emplace_back(binding, info);
    return add_layer(n, l);
}

// Constant layer holding `data` (copied).
int armnnc_add_constant(void* vn, int dtype, int rank, const int32_t* shape, float scale, int32_t zp,
                        const float* scales, int n_scales, int axis, const void* data)
{
    auto* n = static_cast<CNet*>(vn);
    TensorInfo info = info_from(dtype, rank, shape, scale, zp, scales, n_scales, axis, true);
    n->blobs.emplace_back((const uint8_t*)data, (const uint8_t*)data + info.GetNumBytes());
    auto* l = n->net->AddConstantLayer(ConstTensor(info, n->blobs.back().data()));
    l->GetOutputSlot(0).SetTensorInfo(info);
    return add_layer(n, l);
}

void armnnc_connect(void* vn, int from, int from_slot, int to, int to_slot)
{
    auto* n = static_cast<CNet*>(vn);
    n->layers[from]->GetOutputSlot((unsigned)from_slot).Connect(n->layers[to]->GetInputSlot((unsigned)to_slot));
}

void armnnc_set_output_info(void* vn, int layer, int slot, int dtype, int rank, const int32_t* shape, float scale, int32_t zp)
{
    auto* n = static_cast<CNet*>(vn);
    n->layers[layer]->GetOutputSlot((unsigned)slot).SetTensorInfo(info_from(dtype, rank, shape, scale, zp, nullptr, 0, 0, false));
}

int armnnc_add_conv2d(void* vn, int depthwise, int stride_h, int stride_w, int pad_top, int pad_bottom, int pad_left,
                      int pad_right, int dil_h, int dil_w, int bias_enabled, int nchw)
{
    auto* n = static_cast<CNet*>(vn);
    const DataLayout layout = nchw ? DataLayout::NCHW : DataLayout::NHWC;
    if (depthwise) {
        DepthwiseConvolution2dDescriptor d;
        d.m_StrideX = stride_w; d.m_StrideY = stride_h; d.m_PadTop = pad_top; d.m_PadBottom = pad_bottom;
        d.m_PadLeft = pad_left; d.m_PadRight = pad_right; d.m_DilationX = dil_w; d.m_DilationY = dil_h;
        d.m_BiasEnabled = bias_enabled != 0; d.m_DataLayout = layout;
        return add_layer(n, n->net->AddDepthwiseConvolution2dLayer(d));
    }
    Convolution2dDescriptor d;
    d.m_StrideX = stride_w; d.m_StrideY = stride_h; d.m_PadTop = pad_top; d.m_PadBottom = pad_bottom;
    d.m_PadLeft = pad_left; d.m_PadRight = pad_right; d.m_DilationX = dil_w; d.m_DilationY = dil_h;
    d.m_BiasEnabled = bias_enabled != 0; d.m_DataLayout = layout;
    return add_layer(n, n->net->AddConvolution2dLayer(d));
}

int armnnc_add_fully_connected(void* vn, int transpose_w, int bias_enabled)
{
    auto* n = static_cast<CNet*>(vn);
    FullyConnectedDescriptor d;
    d.m_TransposeWeightMatrix = transpose_w != 0; d.m_BiasEnabled = bias_enabled != 0; d.m_ConstantWeights = true;
    return add_layer(n, n->net->AddFullyConnectedLayer(d));
}

int armnnc_add_activation(void* vn, int function, float a, float b)
{
    auto* n = static_cast<CNet*>(vn);
    ActivationDescriptor d;
    d.m_Function = static_cast<ActivationFunction>(function); d.m_A = a; d.m_B = b;
    return add_layer(n, n->net->AddActivationLayer(d));
}

int armnnc_add_pool2d(void* vn, int pool_type, int padding_method, int pool_h, int pool_w, int stride_h, int stride_w,
                      int pad_top, int pad_bottom, int pad_left, int pad_right, int nchw)
{
    auto* n = static_cast<CNet*>(vn);
    Pooling2dDescriptor d;
    d.m_PoolType = static_cast<PoolingAlgorithm>(pool_type); d.m_PaddingMethod = static_cast<PaddingMethod>(padding_method);
    d.m_PoolHeight = pool_h; d.m_PoolWidth = pool_w; d.m_StrideX = stride_w; d.m_StrideY = stride_h;
    d.m_PadTop = pad_top; d.m_PadBottom = pad_bottom; d.m_PadLeft = pad_left; d.m_PadRight = pad_right;
    d.m_OutputShapeRounding = OutputShapeRounding::Floor; d.m_DataLayout = nchw ? DataLayout::NCHW : DataLayout::NHWC;
    return add_layer(n, n->net->AddPooling2dLayer(d));
}

/// strides / dilations: (depth, height, width); pads: (front, back, top, bottom, left, right); NDHWC
int armnnc_add_conv3d(void* vn, const int32_t* strides, const int32_t* pads, const int32_t* dilations, int bias_enabled)
{
    auto* n = static_cast<CNet*>(vn);
    Convolution3dDescriptor d;
    d.m_StrideZ = (unsigned)strides[0]; d.m_StrideY = (unsigned)strides[1]; d.m_StrideX = (unsigned)strides[2];
    d.m_PadFront = (unsigned)pads[0]; d.m_PadBack = (unsigned)pads[1]; d.m_PadTop = (unsigned)pads[2]; d.m_PadBottom = (unsigned)pads[3];
    d.m_PadLeft = (unsigned)pads[4]; d.m_PadRight = (unsigned)pads[5];
    d.m_DilationZ = (unsigned)dilations[0]; d.m_DilationY = (unsigned)dilations[1]; d.m_DilationX = (unsigned)dilations[2];
    d.m_BiasEnabled = bias_enabled != 0; d.m_DataLayout = DataLayout::NDHWC;
    return add_layer(n, n->net->AddConvolution3dLayer(d));
}

int armnnc_add_pool3d(void* vn, int pool_type, int padding_method, const int32_t* pool, const int32_t* strides, const int32_t* pads)
{
    auto* n = static_cast<CNet*>(vn);
    Pooling3dDescriptor d;
    d.m_PoolType = static_cast<PoolingAlgorithm>(pool_type);
    d.m_PaddingMethod = padding_method == 1 ? PaddingMethod::Exclude : PaddingMethod::IgnoreValue;
    d.m_PoolDepth = (unsigned)pool[0]; d.m_PoolHeight = (unsigned)pool[1]; d.m_PoolWidth = (unsigned)pool[2];
    d.m_StrideZ = (unsigned)strides[0]; d.m_StrideY = (unsigned)strides[1]; d.m_StrideX = (unsigned)strides[2];
    d.m_PadFront = (unsigned)pads[0]; d.m_PadBack = (unsigned)pads[1]; d.m_PadTop = (unsigned)pads[2]; d.m_PadBottom = (unsigned)pads[3];
    d.m_PadLeft = (unsigned)pads[4]; d.m_PadRight = (unsigned)pads[5];
    d.m_OutputShapeRounding = OutputShapeRounding::Floor; d.m_DataLayout = DataLayout::NDHWC;
    return add_layer(n, n->net->AddPooling3dLayer(d));
}

int armnnc_add_elementwise_binary(void* vn, int op)
{
    auto* n = static_cast<CNet*>(vn);
    return add_layer(n, n->net->AddElementwiseBinaryLayer(ElementwiseBinaryDescriptor(static_cast<BinaryOperation>(op))));
}

int armnnc_add_normalization(void* vn, int channel_type, unsigned norm_size, float alpha, float beta, float k, int nchw)
{
    auto* n = static_cast<CNet*>(vn);
    NormalizationDescriptor d;
    d.m_NormChannelType = channel_type ? NormalizationAlgorithmChannel::Within : NormalizationAlgorithmChannel::Across;
    d.m_NormMethodType = NormalizationAlgorithmMethod::LocalBrightness;
    d.m_NormSize = norm_size; d.m_Alpha = alpha; d.m_Beta = beta; d.m_K = k;
    d.m_DataLayout = nchw ? DataLayout::NCHW : DataLayout::NHWC;
    return add_layer(n, n->net->AddNormalizationLayer(d));
}

int armnnc_add_scatter_nd(void* vn, int function, int input_enabled)
{
    auto* n = static_cast<CNet*>(vn);
    return add_layer(n, n->net->AddScatterNdLayer(ScatterNdDescriptor(static_cast<ScatterNdFunction>(function), input_enabled != 0)));
}

int armnnc_add_reverse_v2(void* vn)
{
    auto* n = static_cast<CNet*>(vn);
    return add_layer(n, n->net->AddReverseV2Layer());
}

int armnnc_add_gather_nd(void* vn)
{
    auto* n = static_cast<CNet*>(vn);
    return add_layer(n, n->net->AddGatherNdLayer());
}

int armnnc_add_gather(void* vn, int axis)
{
    auto* n = static_cast<CNet*>(vn);
    GatherDescriptor d; d.m_Axis = axis;
    return add_layer(n, n->net->AddGatherLayer(d));
}

/// dtypes / scales / zps / data: mean, variance, beta, gamma (one value per channel each, copied).
int armnnc_add_batch_norm(void* vn, float eps, int nchw, int channels, const int32_t* dtypes, const float* scales,
                          const int32_t* zps, const void* const* data)
{
    auto* n = static_cast<CNet*>(vn);
    BatchNormalizationDescriptor d; d.m_Eps = eps; d.m_DataLayout = nchw ? DataLayout::NCHW : DataLayout::NHWC;
    std::vector<ConstTensor> ts;
    const int32_t shape[1] = {channels};
    for (int i = 0; i < 4; ++i)
    {
        TensorInfo info = info_from(dtypes[i], 1, shape, scales[i], zps[i], nullptr, 0, 0, true);
        n->blobs.emplace_back((const uint8_t*)data[i], (const uint8_t*)data[i] + info.GetNumBytes());
        ts.emplace_back(info, n->blobs.back().data());
    }
    return add_layer(n, n->net->AddBatchNormalizationLayer(d, ts[0], ts[1], ts[2], ts[3]));
}

int armnnc_add_instance_norm(void* vn, float gamma, float beta, float eps, int nchw)
{
    auto* n = static_cast<CNet*>(vn);
    InstanceNormalizationDescriptor d; d.m_Gamma = gamma; d.m_Beta = beta; d.m_Eps = eps;
    d.m_DataLayout = nchw ? DataLayout::NCHW : DataLayout::NHWC;
    return add_layer(n, n->net->AddInstanceNormalizationLayer(d));
}

int armnnc_add_log_softmax(void* vn, float beta, int axis)
{
    auto* n = static_cast<CNet*>(vn);
    LogSoftmaxDescriptor d; d.m_Beta = beta; d.m_Axis = axis;
    return add_layer(n, n->net->AddLogSoftmaxLayer(d));
}

int armnnc_add_l2_normalization(void* vn, float eps, int nchw)
{
    auto* n = static_cast<CNet*>(vn);
    L2NormalizationDescriptor d; d.m_Eps = eps; d.m_DataLayout = nchw ? DataLayout::NCHW : DataLayout::NHWC;
    return add_layer(n, n->net->AddL2NormalizationLayer(d));
}

int armnnc_add_arg_min_max(void* vn, int function, int axis)
{
    auto* n = static_cast<CNet*>(vn);
    ArgMinMaxDescriptor d; d.m_Function = function ? ArgMinMaxFunction::Max : ArgMinMaxFunction::Min; d.m_Axis = axis;
    return add_layer(n, n->net->AddArgMinMaxLayer(d));
}

int armnnc_add_comparison(void* vn, int op)
{
    auto* n = static_cast<CNet*>(vn);
    return add_layer(n, n->net->AddComparisonLayer(ComparisonDescriptor(static_cast<ComparisonOperation>(op))));
}

int armnnc_add_logical_binary(void* vn, int op)
{
    auto* n = static_cast<CNet*>(vn);
    return add_layer(n, n->net->AddLogicalBinaryLayer(LogicalBinaryDescriptor(static_cast<LogicalBinaryOperation>(op))));
}

int armnnc_add_softmax(void* vn, float beta, int axis)
{
    auto* n = static_cast<CNet*>(vn);
    SoftmaxDescriptor d; d.m_Beta = beta; d.m_Axis = axis;
    return add_layer(n, n->net->AddSoftmaxLayer(d));
}

int armnnc_add_mean(void* vn, const int32_t* axes, int n_axes, int keep_dims)
{
    auto* n = static_cast<CNet*>(vn);
    MeanDescriptor d;
    for (int i = 0; i < n_axes; ++i) d.m_Axis.push_back((unsigned)axes[i]);
    d.m_KeepDims = keep_dims != 0;
    return add_layer(n, n->net->AddMeanLayer(d));
}

int armnnc_add_batch_matmul(void* vn, int transpose_x, int transpose_y, int adjoint_x, int adjoint_y)
{
    auto* n = static_cast<CNet*>(vn);
    BatchMatMulDescriptor d(transpose_x != 0, transpose_y != 0, adjoint_x != 0, adjoint_y != 0);
    return add_layer(n, n->net->AddBatchMatMulLayer(d));
}

int armnnc_add_reshape(void* vn, int rank, const int32_t* shape)
{
    auto* n = static_cast<CNet*>(vn);
    unsigned dims[5];
    for (int i = 0; i < rank; ++i) dims[i] = (unsigned)shape[i];
    ReshapeDescriptor d; d.m_TargetShape = TensorShape((unsigned)rank, dims);
    return add_layer(n, n->net->AddReshapeLayer(d));
}

// Lstm (sequence = 0) or UnidirectionalSequenceLstm (sequence = 1) layer on Float32 tensors from a b200k_lstm_params whose
// weight pointers are HOST pointers (copied by Arm NN); only the sizes, weights and option fields are read.
int armnnc_add_lstm(void* vn, const b200k_lstm_params* p, int sequence, int time_major)
{
    auto* n = static_cast<CNet*>(vn);
    const unsigned I = p->input_size, U = p->num_units, O = p->output_size;
    LstmDescriptor d;
    d.m_CifgEnabled = p->w_i2i == nullptr;
    d.m_PeepholeEnabled = p->w_c2f != nullptr;
    d.m_ProjectionEnabled = p->w_proj != nullptr;
    d.m_LayerNormEnabled = p->ln_f != nullptr;
    d.m_ActivationFunc = (uint32_t)p->activation;
    d.m_ClippingThresCell = p->cell_clip; d.m_ClippingThresProj = p->projection_clip;
    d.m_TimeMajor = time_major != 0;
    std::vector<std::unique_ptr<ConstTensor>> keep;
    auto ct = [&](const float* data, TensorShape shape) -> const ConstTensor* {
        if (!data) return nullptr;
        TensorInfo info(shape, DataType::Float32);
        info.SetConstant(true);
        keep.push_back(std::make_unique<ConstTensor>(info, data));
        return keep.back().get();
    };
    LstmInputParams q;
    q.m_InputToInputWeights = ct(p->w_i2i, {U, I}); q.m_InputToForgetWeights = ct(p->w_i2f, {U, I});
    q.m_InputToCellWeights = ct(p->w_i2c, {U, I}); q.m_InputToOutputWeights = ct(p->w_i2o, {U, I});
    q.m_RecurrentToInputWeights = ct(p->w_r2i, {U, O}); q.m_RecurrentToForgetWeights = ct(p->w_r2f, {U, O});
    q.m_RecurrentToCellWeights = ct(p->w_r2c, {U, O}); q.m_RecurrentToOutputWeights = ct(p->w_r2o, {U, O});
    q.m_CellToInputWeights = ct(p->w_c2i, {U}); q.m_CellToForgetWeights = ct(p->w_c2f, {U}); q.m_CellToOutputWeights = ct(p->w_c2o, {U});
    q.m_InputGateBias = ct(p->b_i, {U}); q.m_ForgetGateBias = ct(p->b_f, {U}); q.m_CellBias = ct(p->b_c, {U}); q.m_OutputGateBias = ct(p->b_o, {U});
    q.m_InputLayerNormWeights = ct(p->ln_i, {U}); q.m_ForgetLayerNormWeights = ct(p->ln_f, {U});
    q.m_CellLayerNormWeights = ct(p->ln_c, {U}); q.m_OutputLayerNormWeights = ct(p->ln_o, {U});
    q.m_ProjectionWeights = ct(p->w_proj, {O, U}); q.m_ProjectionBias = ct(p->b_proj, {O});
    try {
        return add_layer(n, sequence ? n->net->AddUnidirectionalSequenceLstmLayer(d, q) : n->net->AddLstmLayer(d, q));
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

// QLstm layer from a b200k_qlstm_params whose weight pointers are HOST pointers (copied by Arm NN); only the weight,
// scale and descriptor fields are read.  Optional weights are null pointers.
int armnnc_add_qlstm(void* vn, const b200k_qlstm_params* p)
{
    auto* n = static_cast<CNet*>(vn);
    const unsigned I = p->input_size, U = p->num_units, O = p->output_size;
    QLstmDescriptor d;
    d.m_CifgEnabled = p->w_i2i == nullptr;
    d.m_PeepholeEnabled = p->w_c2f != nullptr;
    d.m_ProjectionEnabled = p->w_proj != nullptr;
    d.m_LayerNormEnabled = p->ln_f != nullptr;
    d.m_CellClip = p->cell_clip; d.m_ProjectionClip = p->projection_clip;
    d.m_InputIntermediateScale = p->input_intermediate_scale; d.m_ForgetIntermediateScale = p->forget_intermediate_scale;
    d.m_CellIntermediateScale = p->cell_intermediate_scale; d.m_OutputIntermediateScale = p->output_intermediate_scale;
    d.m_HiddenStateScale = p->hidden_state_scale; d.m_HiddenStateZeroPoint = p->hidden_state_zp;
    std::vector<std::unique_ptr<ConstTensor>> keep;
    auto ct = [&](const void* data, TensorShape shape, DataType dt, float scale) -> const ConstTensor* {
        if (!data) return nullptr;
        TensorInfo info(shape, dt, scale, 0);
        info.SetConstant(true);
        keep.push_back(std::make_unique<ConstTensor>(info, data));
        return keep.back().get();
    };
    LstmInputParams q;
    q.m_InputToInputWeights = ct(p->w_i2i, {U, I}, DataType::QSymmS8, p->s_i2i);
    q.m_InputToForgetWeights = ct(p->w_i2f, {U, I}, DataType::QSymmS8, p->s_i2f);
    q.m_InputToCellWeights = ct(p->w_i2c, {U, I}, DataType::QSymmS8, p->s_i2c);
    q.m_InputToOutputWeights = ct(p->w_i2o, {U, I}, DataType::QSymmS8, p->s_i2o);
    q.m_RecurrentToInputWeights = ct(p->w_r2i, {U, O}, DataType::QSymmS8, p->s_r2i);
    q.m_RecurrentToForgetWeights = ct(p->w_r2f, {U, O}, DataType::QSymmS8, p->s_r2f);
    q.m_RecurrentToCellWeights = ct(p->w_r2c, {U, O}, DataType::QSymmS8, p->s_r2c);
    q.m_RecurrentToOutputWeights = ct(p->w_r2o, {U, O}, DataType::QSymmS8, p->s_r2o);
    q.m_CellToInputWeights = ct(p->w_c2i, {U}, DataType::QSymmS16, p->s_c2i);
    q.m_CellToForgetWeights = ct(p->w_c2f, {U}, DataType::QSymmS16, p->s_c2f);
    q.m_CellToOutputWeights = ct(p->w_c2o, {U}, DataType::QSymmS16, p->s_c2o);
    q.m_InputGateBias = ct(p->b_i, {U}, DataType::Signed32, p->s_bi);
    q.m_ForgetGateBias = ct(p->b_f, {U}, DataType::Signed32, p->s_bf);
    q.m_CellBias = ct(p->b_c, {U}, DataType::Signed32, p->s_bc);
    q.m_OutputGateBias = ct(p->b_o, {U}, DataType::Signed32, p->s_bo);
    q.m_InputLayerNormWeights = ct(p->ln_i, {U}, DataType::QSymmS16, p->s_lni);
    q.m_ForgetLayerNormWeights = ct(p->ln_f, {U}, DataType::QSymmS16, p->s_lnf);
    q.m_CellLayerNormWeights = ct(p->ln_c, {U}, DataType::QSymmS16, p->s_lnc);
    q.m_OutputLayerNormWeights = ct(p->ln_o, {U}, DataType::QSymmS16, p->s_lno);
    q.m_ProjectionWeights = ct(p->w_proj, {O, U}, DataType::QSymmS8, p->s_proj);
    q.m_ProjectionBias = ct(p->b_proj, {O}, DataType::Signed32, p->s_bproj);
    try {
        return add_layer(n, n->net->AddQLstmLayer(d, q));
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

// pads: rank pairs (before, after), outermost dimension first
int armnnc_add_shape(void* vn, int rank_only)
{
    auto* n = static_cast<CNet*>(vn);
    return add_layer(n, rank_only ? n->net->AddRankLayer() : n->net->AddShapeLayer());
}

int armnnc_add_cast(void* vn)
{
    auto* n = static_cast<CNet*>(vn);
    return add_layer(n, n->net->AddCastLayer());
}

int armnnc_add_fill(void* vn, float value)
{
    auto* n = static_cast<CNet*>(vn);
    FillDescriptor d; d.m_Value = value;
    return add_layer(n, n->net->AddFillLayer(d));
}

int armnnc_add_floor(void* vn)
{
    auto* n = static_cast<CNet*>(vn);
    return add_layer(n, n->net->AddFloorLayer());
}

int armnnc_add_pad(void* vn, int rank, const int32_t* pads, float pad_value, int mode)
{
    auto* n = static_cast<CNet*>(vn);
    PadDescriptor d;
    for (int i = 0; i < rank; ++i) d.m_PadList.emplace_back((unsigned)pads[2 * i], (unsigned)pads[2 * i + 1]);
    d.m_PadValue = pad_value;
    d.m_PaddingMode = mode == 1 ? PaddingMode::Reflect : mode == 2 ? PaddingMode::Symmetric : PaddingMode::Constant;
    return add_layer(n, n->net->AddPadLayer(d));
}

// origins: n_views x rank coordinates of each input's block in the output
int armnnc_add_concat(void* vn, int n_views, int rank, const int32_t* origins)
{
    auto* n = static_cast<CNet*>(vn);
    OriginsDescriptor d((uint32_t)n_views, (uint32_t)rank);
    for (int v = 0; v < n_views; ++v)
        for (int i = 0; i < rank; ++i) d.SetViewOriginCoord((uint32_t)v, (uint32_t)i, (uint32_t)origins[v * rank + i]);
    return add_layer(n, n->net->AddConcatLayer(d));
}

// origins / sizes: n_views x rank
int armnnc_add_splitter(void* vn, int n_views, int rank, const int32_t* origins, const int32_t* sizes)
{
    auto* n = static_cast<CNet*>(vn);
    ViewsDescriptor d((uint32_t)n_views, (uint32_t)rank);
    for (int v = 0; v < n_views; ++v)
        for (int i = 0; i < rank; ++i) {
            d.SetViewOriginCoord((uint32_t)v, (uint32_t)i, (uint32_t)origins[v * rank + i]);
            d.SetViewSize((uint32_t)v, (uint32_t)i, (uint32_t)sizes[v * rank + i]);
        }
    return add_layer(n, n->net->AddSplitterLayer(d));
}

int armnnc_add_permute(void* vn, int rank, const int32_t* mappings, int transpose)
{
    auto* n = static_cast<CNet*>(vn);
    unsigned m[6] = {0, 0, 0, 0, 0, 0};
    for (int i = 0; i < rank && i < 6; ++i) m[i] = (unsigned)mappings[i];
    try {
        const PermutationVector pv(m, (unsigned)rank);
        if (transpose) return add_layer(n, n->net->AddTransposeLayer(TransposeDescriptor(pv)));
        return add_layer(n, n->net->AddPermuteLayer(PermuteDescriptor(pv)));
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

int armnnc_add_strided_slice(void* vn, int rank, const int32_t* begin, const int32_t* end, const int32_t* stride,
                             int begin_mask, int end_mask, int shrink_axis_mask, int ellipsis_mask, int new_axis_mask)
{
    auto* n = static_cast<CNet*>(vn);
    StridedSliceDescriptor d;
    d.m_EllipsisMask = ellipsis_mask; d.m_NewAxisMask = new_axis_mask;
    d.m_Begin.assign(begin, begin + rank);
    d.m_End.assign(end, end + rank);
    d.m_Stride.assign(stride, stride + rank);
    d.m_BeginMask = begin_mask; d.m_EndMask = end_mask; d.m_ShrinkAxisMask = shrink_axis_mask;
    return add_layer(n, n->net->AddStridedSliceLayer(d));
}

int armnnc_add_slice(void* vn, int rank, const int32_t* begin, const int32_t* size)
{
    auto* n = static_cast<CNet*>(vn);
    SliceDescriptor d;
    d.m_Begin.assign(begin, begin + rank);
    d.m_Size.assign(size, size + rank);
    return add_layer(n, n->net->AddSliceLayer(d));
}

// weights [OC, KH, KW, C] and the optional bias travel as ConstTensor arguments of the layer (INetwork.hpp)
int armnnc_add_transpose_conv2d(void* vn, int stride_h, int stride_w, int pad_top, int pad_bottom, int pad_left, int pad_right,
                                int w_dtype, const int32_t* w_shape, float w_scale, int32_t w_zp, const float* w_scales, int n_w_scales,
                                const void* w_data, const void* b_data, float b_scale, const float* b_scales, int n_b_scales, int nchw)
{
    auto* n = static_cast<CNet*>(vn);
    TransposeConvolution2dDescriptor d;
    d.m_StrideY = (uint32_t)stride_h; d.m_StrideX = (uint32_t)stride_w;
    d.m_PadTop = (uint32_t)pad_top; d.m_PadBottom = (uint32_t)pad_bottom; d.m_PadLeft = (uint32_t)pad_left; d.m_PadRight = (uint32_t)pad_right;
    d.m_BiasEnabled = b_data != nullptr;
    d.m_DataLayout = nchw ? DataLayout::NCHW : DataLayout::NHWC;
    TensorInfo wi = info_from(w_dtype, 4, w_shape, w_scale, w_zp, w_scales, n_w_scales, 0, true);
    n->blobs.emplace_back((const uint8_t*)w_data, (const uint8_t*)w_data + wi.GetNumBytes());
    ConstTensor weights(wi, n->blobs.back().data());
    Optional<ConstTensor> bias;
    if (b_data) {
        const int32_t bshape[1] = {w_shape[0]};
        TensorInfo bi = info_from(3 /* Signed32 */, 1, bshape, b_scale, 0, b_scales, n_b_scales, 0, true);
        n->blobs.emplace_back((const uint8_t*)b_data, (const uint8_t*)b_data + bi.GetNumBytes());
        bias = Optional<ConstTensor>(ConstTensor(bi, n->blobs.back().data()));
    }
    try {
        return add_layer(n, n->net->AddTransposeConvolution2dLayer(d, weights, bias));
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

int armnnc_add_depth_to_space(void* vn, int block, int nchw, int inverse)
{
    auto* n = static_cast<CNet*>(vn);
    SpaceToDepthDescriptor d;              // (DepthToSpaceDescriptor is an alias of it)
    d.m_BlockSize = (unsigned)block;
    d.m_DataLayout = nchw ? DataLayout::NCHW : DataLayout::NHWC;
    return add_layer(n, inverse ? n->net->AddSpaceToDepthLayer(d) : n->net->AddDepthToSpaceLayer(d));
}

/// edges: (before, after) per spatial dimension, flattened.  inverse = 0: BatchToSpaceNd with crops; 1: SpaceToBatchNd with padding.
int armnnc_add_batch_to_space(void* vn, const int32_t* block, const int32_t* edges, int n_spatial, int nchw, int inverse)
{
    auto* n = static_cast<CNet*>(vn);
    std::vector<unsigned int> blockShape;
    std::vector<std::pair<unsigned int, unsigned int>> pairs;
    for (int i = 0; i < n_spatial; ++i)
    {
        blockShape.push_back(static_cast<unsigned int>(block[i]));
        pairs.emplace_back(static_cast<unsigned int>(edges[2 * i]), static_cast<unsigned int>(edges[2 * i + 1]));
    }
    if (inverse)
    {
        SpaceToBatchNdDescriptor d(blockShape, pairs);
        d.m_DataLayout = nchw ? DataLayout::NCHW : DataLayout::NHWC;
        return add_layer(n, n->net->AddSpaceToBatchNdLayer(d));
    }
    BatchToSpaceNdDescriptor d(blockShape, pairs);
    d.m_DataLayout = nchw ? DataLayout::NCHW : DataLayout::NHWC;
    return add_layer(n, n->net->AddBatchToSpaceNdLayer(d));
}

int armnnc_add_tile(void* vn, const int32_t* multiples, int rank)
{
    auto* n = static_cast<CNet*>(vn);
    TileDescriptor d;
    d.m_Multiples.assign(multiples, multiples + rank);
    return add_layer(n, n->net->AddTileLayer(d));
}

int armnnc_add_broadcast_to(void* vn, const int32_t* shape, int rank)
{
    auto* n = static_cast<CNet*>(vn);
    unsigned dims[6] = {0, 0, 0, 0, 0, 0};
    for (int i = 0; i < rank && i < 6; ++i) dims[i] = (unsigned)shape[i];
    BroadcastToDescriptor d;
    d.m_BroadcastToShape = TensorShape((unsigned)rank, dims);
    return add_layer(n, n->net->AddBroadcastToLayer(d));
}

int armnnc_add_channel_shuffle(void* vn, int axis, int groups)
{
    auto* n = static_cast<CNet*>(vn);
    ChannelShuffleDescriptor d;
    d.m_Axis = (uint32_t)axis; d.m_NumGroups = (uint32_t)groups;
    return add_layer(n, n->net->AddChannelShuffleLayer(d));
}

int armnnc_add_stack(void* vn, int axis, int num_inputs, int rank, const int32_t* input_shape)
{
    auto* n = static_cast<CNet*>(vn);
    unsigned dims[6] = {1, 1, 1, 1, 1, 1};
    for (int i = 0; i < rank && i < 6; ++i) dims[i] = (unsigned)input_shape[i];
    StackDescriptor d((uint32_t)axis, (uint32_t)num_inputs, TensorShape((unsigned)rank, dims));
    return add_layer(n, n->net->AddStackLayer(d));
}

int armnnc_add_elementwise_unary(void* vn, int operation)
{
    auto* n = static_cast<CNet*>(vn);
    return add_layer(n, n->net->AddElementwiseUnaryLayer(ElementwiseUnaryDescriptor(static_cast<UnaryOperation>(operation))));
}

int armnnc_add_prelu(void* vn)
{
    auto* n = static_cast<CNet*>(vn);
    return add_layer(n, n->net->AddPreluLayer());
}

int armnnc_add_reduce(void* vn, const int32_t* axes, int n_axes, int operation, int keep_dims)
{
    auto* n = static_cast<CNet*>(vn);
    ReduceDescriptor d;
    for (int i = 0; i < n_axes; ++i) d.m_vAxis.push_back((uint32_t)axes[i]);
    d.m_ReduceOperation = static_cast<ReduceOperation>(operation);
    d.m_KeepDims = keep_dims != 0;
    return add_layer(n, n->net->AddReduceLayer(d));
}

int armnnc_add_resize(void* vn, int height, int width, int method, int align_corners, int half_pixel_centers, int nchw)
{
    auto* n = static_cast<CNet*>(vn);
    ResizeDescriptor d;
    d.m_TargetHeight = (uint32_t)height; d.m_TargetWidth = (uint32_t)width;
    d.m_Method = method == 0 ? ResizeMethod::Bilinear : ResizeMethod::NearestNeighbor;
    d.m_DataLayout = nchw ? DataLayout::NCHW : DataLayout::NHWC;
    d.m_AlignCorners = align_corners != 0; d.m_HalfPixelCenters = half_pixel_centers != 0;
    return add_layer(n, n->net->AddResizeLayer(d));
}

int armnnc_add_quantize(void* vn)   { auto* n = static_cast<CNet*>(vn); return add_layer(n, n->net->AddQuantizeLayer()); }
int armnnc_add_dequantize(void* vn) { auto* n = static_cast<CNet*>(vn); return add_layer(n, n->net->AddDequantizeLayer()); }

int armnnc_add_output(void* vn, int binding, int from_layer, int from_slot)
{
    auto* n = static_cast<CNet*>(vn);
    auto* l = n->net->AddOutputLayer(binding);
    n->layers[from_layer]->GetOutputSlot((unsigned)from_slot).Connect(l->GetInputSlot(0));
    n->outputs.emplace_back(binding, n->layers[from_layer]->GetOutputSlot((unsigned)from_slot).GetTensorInfo());
    return add_layer(n, l);
}

// Optimize for the comma-separated backend preference list and load.  device_id >= 0 is passed to
// the B200Acc backend as ModelOption "DeviceId".  flags: bit 0 = profiling, bit 1 = load with
// INetworkProperties{MemorySource::Malloc, MemorySource::Malloc} (EnqueueWorkload imports the caller's buffers).
void* armnnc_load(void* vr, void* vn, const char* backends, int device_id, int flags)
{
    const int profiling = flags & 1;
    const MemorySource io = (flags & 2) ? MemorySource::Malloc : MemorySource::Undefined;
    auto* r = static_cast<CRuntime*>(vr);
    auto* n = static_cast<CNet*>(vn);
    try {
        std::vector<BackendId> prefs;
        std::string s(backends);
        size_t pos = 0;
        while (pos <= s.size()) {
            size_t c = s.find(',', pos);
            if (c == std::string::npos) c = s.size();
            if (c > pos) prefs.emplace_back(s.substr(pos, c - pos));
            pos = c + 1;
        }
        OptimizerOptionsOpaque oo;
        if (device_id >= 0) oo.AddModelOption(BackendOptions("B200Acc", {{"DeviceId", device_id}}));
        oo.SetProfilingEnabled(profiling != 0);
        if (flags & 2) { oo.SetImportEnabled(true); oo.SetExportEnabled(true); }
        std::vector<std::string> messages;
        IOptimizedNetworkPtr opt = Optimize(*n->net, prefs, r->rt->GetDeviceSpec(), oo, Optional<std::vector<std::string>&>(messages));
        if (!opt) { g_err = "Optimize returned null"; for (auto& m : messages) g_err += "; " + m; return nullptr; }
        auto* l = new CLoaded;
        l->rt = r;
        std::string err;
        INetworkProperties props(io, io, profiling != 0);
        if (r->rt->LoadNetwork(l->id, std::move(opt), err, props) != Status::Success) {
            g_err = "LoadNetwork failed: " + err;
            delete l;
            return nullptr;
        }
        l->inputs = n->inputs; l->outputs = n->outputs;
        return l;
    } catch (const std::exception& e) { g_err = e.what(); return nullptr; }
}

// Optimize only (no device needed): writes one "LayerType name" line per layer of the optimized graph, in
// execution order, into buf; returns the number of bytes needed, 0 on failure.
size_t armnnc_optimized_layers(void* vr, void* vn, const char* backends, char* buf, size_t cap)
{
    auto* r = static_cast<CRuntime*>(vr);
    auto* n = static_cast<CNet*>(vn);
    struct Lister : IStrategy {
        std::ostringstream os;
        void ExecuteStrategy(const IConnectableLayer* layer, const BaseDescriptor&, const std::vector<ConstTensor>&,
                             const char* name, const LayerBindingId) override
        { os << GetLayerTypeAsCString(layer->GetType()) << " " << (name ? name : "") << "\n"; }
    } lister;
    try {
        std::vector<std::string> messages;
        IOptimizedNetworkPtr opt = Optimize(*n->net, {BackendId(backends)}, r->rt->GetDeviceSpec(), OptimizerOptionsOpaque(),
                                            Optional<std::vector<std::string>&>(messages));
        if (!opt) { g_err = "Optimize returned null"; for (auto& m : messages) g_err += "; " + m; return 0; }
        opt->ExecuteStrategy(lister);
    } catch (const std::exception& e) { g_err = e.what(); return 0; }
    std::string s = lister.os.str();
    if (buf && cap) { size_t k = std::min(cap - 1, s.size()); std::memcpy(buf, s.data(), k); buf[k] = 0; }
    return s.size() + 1;
}

void armnnc_unload(void* vl)
{
    auto* l = static_cast<CLoaded*>(vl);
    l->rt->rt->UnloadNetwork(l->id);
    delete l;
}

// inputs / outputs: arrays of host pointers in the order the Input / Output layers were added.
int armnnc_enqueue(void* vl, const void* const* inputs, void* const* outputs)
{
    auto* l = static_cast<CLoaded*>(vl);
    try {
        InputTensors in;
        OutputTensors out;
        for (size_t i = 0; i < l->inputs.size(); ++i) {
            TensorInfo info = l->inputs[i].second;
            info.SetConstant(true);
            in.emplace_back(l->inputs[i].first, ConstTensor(info, inputs[i]));
        }
        for (size_t i = 0; i < l->outputs.size(); ++i)
            out.emplace_back(l->outputs[i].first, Tensor(l->outputs[i].second, outputs[i]));
        return l->rt->rt->EnqueueWorkload(l->id, in, out) == Status::Success ? 0 : -1;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

// The same through the pre-import API: the first call (and any call with other pointers) imports the buffers with
// IRuntime::ImportInputs / ImportOutputs(MemorySource::Malloc); EnqueueWorkload then runs on the imported ids only.
int armnnc_enqueue_preimported(void* vl, const void* const* inputs, void* const* outputs)
{
    auto* l = static_cast<CLoaded*>(vl);
    try {
        std::vector<const void*> in_ptrs(inputs, inputs + l->inputs.size());
        std::vector<void*> out_ptrs(outputs, outputs + l->outputs.size());
        if (in_ptrs != l->pre_in_ptrs || out_ptrs != l->pre_out_ptrs) {
            InputTensors in;
            OutputTensors out;
            for (size_t i = 0; i < l->inputs.size(); ++i) {
                TensorInfo info = l->inputs[i].second;
                info.SetConstant(true);
                in.emplace_back(l->inputs[i].first, ConstTensor(info, inputs[i]));
            }
            for (size_t i = 0; i < l->outputs.size(); ++i)
                out.emplace_back(l->outputs[i].first, Tensor(l->outputs[i].second, outputs[i]));
            l->pre_in = l->rt->rt->ImportInputs(l->id, in, MemorySource::Malloc);
            l->pre_out = l->rt->rt->ImportOutputs(l->id, out, MemorySource::Malloc);
            if (l->pre_in.size() != l->inputs.size() || l->pre_out.size() != l->outputs.size()) {
                g_err = "ImportInputs / ImportOutputs did not import every tensor";
                return -2;
            }
            l->pre_in_ptrs = in_ptrs; l->pre_out_ptrs = out_ptrs;
        }
        return l->rt->rt->EnqueueWorkload(l->id, {}, {}, l->pre_in, l->pre_out) == Status::Success ? 0 : -1;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

// Writes the profiler's JSON (per-workload timings) into buf; returns the number of bytes needed.
size_t armnnc_profile_json(void* vl, char* buf, size_t cap)
{
    auto* l = static_cast<CLoaded*>(vl);
    auto prof = l->rt->rt->GetProfiler(l->id);
    if (!prof) return 0;
    std::ostringstream os;
    prof->Print(os);
    std::string s = os.str();
    if (buf && cap) { size_t k = std::min(cap - 1, s.size()); std::memcpy(buf, s.data(), k); buf[k] = 0; }
    return s.size() + 1;
}

}  // extern "C"
