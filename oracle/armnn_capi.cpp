// TEST INFRASTRUCTURE ONLY — a C binding over the unmodified Arm NN reference (oracle/_ref/libarmnn.so)
// so that Python tests and the CPU-baseline leg of the benchmark can run the *real* CpuRef workloads.
//
// Part 1 (cpuref_*): workload-level execution, the way the reference's own layer tests drive a backend
// (src/backends/backendsCommon/test/layerTests/Conv2dTestImpl.cpp:3562-3669): build TensorInfos and a
// QueueDescriptor by hand, RefWorkloadFactory::CreateWorkload, Execute.  The functions take the same
// parameter structs as include/b200k.h, with HOST pointers, so a test hands one struct to the CPU
// restatement, to real CpuRef and (with device pointers) to the CUDA library.
//
// Part 2 (armnnc_*): a minimal graph-level binding: INetwork -> Optimize(backend list) -> LoadNetwork ->
// EnqueueWorkload, for any registered backend id ("CpuRef", or "B200Acc" loaded as a dynamic backend).
#include <armnn/ArmNN.hpp>
#include <armnn/BackendRegistry.hpp>
#include <armnn/backends/TensorHandle.hpp>
#include <armnn/backends/WorkloadData.hpp>
#include <armnn/backends/WorkloadFactory.hpp>
#include <reference/RefWorkloadFactory.hpp>
#include <reference/RefTensorHandleFactory.hpp>
#include <reference/RefMemoryManager.hpp>

#include <algorithm>
#include <chrono>
#include <sstream>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../include/b200k.h"

using namespace armnn;

static thread_local std::string g_err;
extern "C" const char* cpuref_last_error() { return g_err.c_str(); }

namespace {

DataType act_type(int dt)
{
    switch (dt) {
        case B200K_U8:  return DataType::QAsymmU8;
        case B200K_S8:  return DataType::QAsymmS8;
        case B200K_S16: return DataType::QSymmS16;
        case B200K_S32: return DataType::Signed32;
        default:        return DataType::Float32;
    }
}

size_t elem_bytes(int dt) { return dt == B200K_U8 || dt == B200K_S8 ? 1 : dt == B200K_S16 ? 2 : 4; }

// TensorInfo of an operand; per-axis scales (weights / bias) when t.scales != NULL.
TensorInfo make_info(const b200k_qtensor& t, const TensorShape& shape, unsigned axis_dim, unsigned n_axis,
                     bool constant)
{
    TensorInfo info(shape, act_type(t.dtype));
    if (t.scales) {
        if (t.dtype == B200K_S8) info.SetDataType(DataType::QSymmS8);
        info.SetQuantizationScales(std::vector<float>(t.scales, t.scales + n_axis));
        info.SetQuantizationDim(Optional<unsigned int>(axis_dim));
    } else if (t.dtype != B200K_F32) {
        info.SetQuantizationScale(t.scale);
        info.SetQuantizationOffset(t.zero_point);
    }
    info.SetConstant(constant);
    return info;
}

struct Harness {
    RefWorkloadFactory factory;
    RefTensorHandleFactory thf{std::make_shared<RefMemoryManager>()};
    std::vector<std::unique_ptr<ITensorHandle>> handles;
    WorkloadInfo winfo;

    ITensorHandle* in(QueueDescriptor& d, const TensorInfo& info, const void* data)
    {
        auto h = thf.CreateTensorHandle(info);
        h->Allocate();
        std::memcpy(h->Map(), data, info.GetNumBytes());
        h->Unmap();
        d.m_Inputs.push_back(h.get());
        winfo.m_InputTensorInfos.push_back(info);
        handles.push_back(std::move(h));
        return handles.back().get();
    }
    ITensorHandle* out(QueueDescriptor& d, const TensorInfo& info)
    {
        auto h = thf.CreateTensorHandle(info);
        h->Allocate();
        d.m_Outputs.push_back(h.get());
        winfo.m_OutputTensorInfos.push_back(info);
        handles.push_back(std::move(h));
        return handles.back().get();
    }
    void run(LayerType type, const QueueDescriptor& d)
    {
        auto wl = factory.CreateWorkload(type, d, winfo);
        if (!wl) throw RuntimeException("RefWorkloadFactory returned no workload");
        wl->PostAllocationConfigure();
        wl->Execute();
    }
};

void copy_out(ITensorHandle* h, void* dst, size_t bytes)
{
    std::memcpy(dst, h->Map(), bytes);
    h->Unmap();
}

// Optional separate Activation workload on the output, as CpuRef has no fused activations.
void run_activation(int kind, float a, float b, const TensorInfo& info, void* data)
{
    if (kind == 0) return;
    Harness h;
    ActivationQueueDescriptor d;
    d.m_Parameters.m_Function = kind == 1 ? ActivationFunction::ReLu : ActivationFunction::BoundedReLu;
    d.m_Parameters.m_A = a;
    d.m_Parameters.m_B = b;
    h.in(d, info, data);
    auto* o = h.out(d, info);
    h.run(LayerType::Activation, d);
    copy_out(o, data, info.GetNumBytes());
}

template <typename F>
int guarded(F&& f)
{
    try { f(); return 0; }
    catch (const std::exception& e) { g_err = e.what(); return -1; }
}

}  // namespace

extern "C" int cpuref_conv2d_q8(const b200k_conv2d_params* p, int depthwise, int act_kind, float act_a, float act_b)
{
    return guarded([&] {
        Harness h;
        const unsigned N = p->n, H = p->h, W = p->wd, C = p->c, OH = p->oh, OW = p->ow, OC = p->oc, KH = p->kh, KW = p->kw;
        TensorInfo xi = make_info(p->x, TensorShape({N, H, W, C}), 0, 0, false);
        TensorInfo wi = depthwise ? make_info(p->w, TensorShape({1, KH, KW, OC}), 3, OC, true)
                                  : make_info(p->w, TensorShape({OC, KH, KW, C}), 0, OC, true);
        TensorInfo yi = make_info(p->y, TensorShape({N, OH, OW, OC}), 0, 0, false);
        // pad_bottom / pad_right only influence shape inference, which the caller has already done
        auto fill = [&](auto& desc) {
            desc.m_PadTop = p->pad_top; desc.m_PadLeft = p->pad_left;
            desc.m_PadBottom = 0; desc.m_PadRight = 0;
            desc.m_StrideX = p->stride_w; desc.m_StrideY = p->stride_h;
            desc.m_DilationX = p->dil_w; desc.m_DilationY = p->dil_h;
            desc.m_BiasEnabled = p->bias.data != nullptr;
            desc.m_DataLayout = DataLayout::NHWC;
        };
        ITensorHandle* o = nullptr;
        if (depthwise) {
            DepthwiseConvolution2dQueueDescriptor d;
            fill(d.m_Parameters);
            h.in(d, xi, p->x.data);
            h.in(d, wi, p->w.data);
            if (p->bias.data) h.in(d, make_info(p->bias, TensorShape({OC}), 0, OC, true), p->bias.data);
            o = h.out(d, yi);
            h.run(LayerType::DepthwiseConvolution2d, d);
        } else {
            Convolution2dQueueDescriptor d;
            fill(d.m_Parameters);
            h.in(d, xi, p->x.data);
            h.in(d, wi, p->w.data);
            if (p->bias.data) h.in(d, make_info(p->bias, TensorShape({OC}), 0, OC, true), p->bias.data);
            o = h.out(d, yi);
            h.run(LayerType::Convolution2d, d);
        }
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
        run_activation(act_kind, act_a, act_b, yi, const_cast<void*>(p->y.data));
    });
}

extern "C" int cpuref_fully_connected_q8(const b200k_fc_params* p, int act_kind, float act_a, float act_b)
{
    return guarded([&] {
        Harness h;
        const unsigned M = p->m, K = p->k, N = p->n;
        TensorInfo xi = make_info(p->x, TensorShape({M, K}), 0, 0, false);
        TensorInfo wi = p->transpose_w ? make_info(p->w, TensorShape({N, K}), 0, N, true)
                                       : make_info(p->w, TensorShape({K, N}), 1, N, true);
        TensorInfo yi = make_info(p->y, TensorShape({M, N}), 0, 0, false);
        FullyConnectedQueueDescriptor d;
        d.m_Parameters.m_BiasEnabled = p->bias.data != nullptr;
        d.m_Parameters.m_TransposeWeightMatrix = p->transpose_w != 0;
        d.m_Parameters.m_ConstantWeights = true;
        h.in(d, xi, p->x.data);
        h.in(d, wi, p->w.data);
        if (p->bias.data) h.in(d, make_info(p->bias, TensorShape({N}), 0, N, true), p->bias.data);
        auto* o = h.out(d, yi);
        h.run(LayerType::FullyConnected, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
        run_activation(act_kind, act_a, act_b, yi, const_cast<void*>(p->y.data));
    });
}

extern "C" int cpuref_batch_matmul_q8(const b200k_bmm_params* p)
{
    return guarded([&] {
        Harness h;
        const unsigned B = p->batch, M = p->m, K = p->k, N = p->n;
        const unsigned bx = p->batch_stride_x == 0 ? 1 : B, by = p->batch_stride_y == 0 ? 1 : B;
        TensorInfo xi = make_info(p->x, p->transpose_x ? TensorShape({bx, K, M}) : TensorShape({bx, M, K}), 0, 0, false);
        TensorInfo yi = make_info(p->y, p->transpose_y ? TensorShape({by, N, K}) : TensorShape({by, K, N}), 0, 0, false);
        TensorInfo oi = make_info(p->out, TensorShape({B, M, N}), 0, 0, false);
        BatchMatMulQueueDescriptor d;
        d.m_Parameters.m_TransposeX = p->transpose_x != 0;
        d.m_Parameters.m_TransposeY = p->transpose_y != 0;
        h.in(d, xi, p->x.data);
        h.in(d, yi, p->y.data);
        auto* o = h.out(d, oi);
        h.run(LayerType::BatchMatMul, d);
        copy_out(o, const_cast<void*>(p->out.data), oi.GetNumBytes());
    });
}

extern "C" int cpuref_pool2d_q8(const b200k_pool2d_params* p)
{
    return guarded([&] {
        Harness h;
        const unsigned N = p->n, H = p->h, W = p->wd, C = p->c, OH = p->oh, OW = p->ow;
        TensorInfo xi = make_info(p->x, TensorShape({N, H, W, C}), 0, 0, false);
        TensorInfo yi = make_info(p->y, TensorShape({N, OH, OW, C}), 0, 0, false);
        Pooling2dQueueDescriptor d;
        auto& q = d.m_Parameters;
        q.m_PoolType = static_cast<PoolingAlgorithm>(p->pool_type);
        q.m_PaddingMethod = static_cast<PaddingMethod>(p->padding_method);
        q.m_PoolHeight = p->pool_h; q.m_PoolWidth = p->pool_w; q.m_StrideX = p->stride_w; q.m_StrideY = p->stride_h;
        q.m_PadTop = p->pad_top; q.m_PadBottom = p->pad_bottom; q.m_PadLeft = p->pad_left; q.m_PadRight = p->pad_right;
        q.m_OutputShapeRounding = OutputShapeRounding::Floor;
        q.m_DataLayout = DataLayout::NHWC;
        h.in(d, xi, p->x.data);
        auto* o = h.out(d, yi);
        h.run(LayerType::Pooling2d, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_mean_hw_q8(const b200k_mean_params* p)
{
    return guarded([&] {
        Harness h;
        const unsigned N = p->n, H = p->h, W = p->wd, C = p->c;
        TensorInfo xi = make_info(p->x, TensorShape({N, H, W, C}), 0, 0, false);
        TensorInfo yi = make_info(p->y, TensorShape({N, C}), 0, 0, false);
        MeanQueueDescriptor d;
        d.m_Parameters.m_Axis = {1, 2};
        d.m_Parameters.m_KeepDims = false;
        h.in(d, xi, p->x.data);
        auto* o = h.out(d, yi);
        h.run(LayerType::Mean, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_eltwise_q8(const b200k_eltwise_params* p, int act_kind, float act_a, float act_b)
{
    return guarded([&] {
        Harness h;
        auto shape = [&](const int32_t* s) {
            unsigned dims[4];
            for (int i = 0; i < p->rank; ++i) dims[i] = (unsigned)s[i];
            return TensorShape((unsigned)p->rank, dims);
        };
        TensorInfo ai = make_info(p->a, shape(p->shape_a), 0, 0, false);
        TensorInfo bi = make_info(p->b, shape(p->shape_b), 0, 0, false);
        TensorInfo oi = make_info(p->out, shape(p->shape_out), 0, 0, false);
        ElementwiseBinaryQueueDescriptor d;
        d.m_Parameters.m_Operation = static_cast<BinaryOperation>(p->op);
        h.in(d, ai, p->a.data);
        h.in(d, bi, p->b.data);
        auto* o = h.out(d, oi);
        h.run(LayerType::ElementwiseBinary, d);
        copy_out(o, const_cast<void*>(p->out.data), oi.GetNumBytes());
        run_activation(act_kind, act_a, act_b, oi, const_cast<void*>(p->out.data));
    });
}

extern "C" int cpuref_activation_q8(const b200k_activation_params* p)
{
    return guarded([&] {
        Harness h;
        TensorInfo xi = make_info(p->x, TensorShape({(unsigned)p->count}), 0, 0, false);
        TensorInfo yi = make_info(p->y, TensorShape({(unsigned)p->count}), 0, 0, false);
        ActivationQueueDescriptor d;
        d.m_Parameters.m_Function = static_cast<ActivationFunction>(p->function);
        d.m_Parameters.m_A = p->a;
        d.m_Parameters.m_B = p->b;
        h.in(d, xi, p->x.data);
        auto* o = h.out(d, yi);
        h.run(LayerType::Activation, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_softmax_q8(const b200k_softmax_params* p)
{
    return guarded([&] {
        Harness h;
        TensorShape s({(unsigned)p->outer, (unsigned)p->axis_size, (unsigned)p->inner});
        TensorInfo xi = make_info(p->x, s, 0, 0, false);
        TensorInfo yi = make_info(p->y, s, 0, 0, false);
        SoftmaxQueueDescriptor d;
        d.m_Parameters.m_Beta = p->beta;
        d.m_Parameters.m_Axis = 1;
        h.in(d, xi, p->x.data);
        auto* o = h.out(d, yi);
        h.run(LayerType::Softmax, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_convert_q(const b200k_convert_params* p)
{
    return guarded([&] {
        Harness h;
        TensorInfo xi = make_info(p->x, TensorShape({(unsigned)p->count}), 0, 0, false);
        TensorInfo yi = make_info(p->y, TensorShape({(unsigned)p->count}), 0, 0, false);
        ITensorHandle* o = nullptr;
        if (p->y.dtype == B200K_F32) {
            DequantizeQueueDescriptor d;
            h.in(d, xi, p->x.data);
            o = h.out(d, yi);
            h.run(LayerType::Dequantize, d);
        } else {
            QuantizeQueueDescriptor d;
            h.in(d, xi, p->x.data);
            o = h.out(d, yi);
            h.run(LayerType::Quantize, d);
        }
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_qlstm_step(const b200k_qlstm_params* p)
{
    return guarded([&] {
        Harness h;
        const unsigned B = p->batch, I = p->input_size, U = p->num_units, O = p->output_size;
        TensorInfo xi({B, I}, DataType::QAsymmS8, p->input_scale, p->input_zp);
        TensorInfo hi({B, O}, DataType::QAsymmS8, p->output_state_scale, p->output_state_zp);
        TensorInfo ci({B, U}, DataType::QSymmS16, p->cell_state_scale, 0);
        TensorInfo oi({B, O}, DataType::QAsymmS8, p->output_scale, p->output_zp);
        QLstmQueueDescriptor d;
        auto& q = d.m_Parameters;
        q.m_CifgEnabled = p->w_i2i == nullptr;
        q.m_PeepholeEnabled = p->w_c2f != nullptr;
        q.m_ProjectionEnabled = p->w_proj != nullptr;
        q.m_LayerNormEnabled = p->ln_f != nullptr;
        q.m_CellClip = p->cell_clip; q.m_ProjectionClip = p->projection_clip;
        q.m_InputIntermediateScale = p->input_intermediate_scale;
        q.m_ForgetIntermediateScale = p->forget_intermediate_scale;
        q.m_CellIntermediateScale = p->cell_intermediate_scale;
        q.m_OutputIntermediateScale = p->output_intermediate_scale;
        q.m_HiddenStateScale = p->hidden_state_scale; q.m_HiddenStateZeroPoint = p->hidden_state_zp;

        std::vector<std::unique_ptr<ScopedTensorHandle>> keep;
        auto weight = [&](const void* data, TensorShape shape, DataType dt, float scale) -> const ConstTensorHandle* {
            if (!data) return nullptr;
            TensorInfo info(shape, dt, scale, 0);
            info.SetConstant(true);
            auto t = std::make_unique<ScopedTensorHandle>(info);
            t->Allocate();
            std::memcpy(t->GetTensor<void>(), data, info.GetNumBytes());
            keep.push_back(std::move(t));
            return keep.back().get();
        };
        d.m_InputToInputWeights  = weight(p->w_i2i, {U, I}, DataType::QSymmS8, p->s_i2i);
        d.m_InputToForgetWeights = weight(p->w_i2f, {U, I}, DataType::QSymmS8, p->s_i2f);
        d.m_InputToCellWeights   = weight(p->w_i2c, {U, I}, DataType::QSymmS8, p->s_i2c);
        d.m_InputToOutputWeights = weight(p->w_i2o, {U, I}, DataType::QSymmS8, p->s_i2o);
        d.m_RecurrentToInputWeights  = weight(p->w_r2i, {U, O}, DataType::QSymmS8, p->s_r2i);
        d.m_RecurrentToForgetWeights = weight(p->w_r2f, {U, O}, DataType::QSymmS8, p->s_r2f);
        d.m_RecurrentToCellWeights   = weight(p->w_r2c, {U, O}, DataType::QSymmS8, p->s_r2c);
        d.m_RecurrentToOutputWeights = weight(p->w_r2o, {U, O}, DataType::QSymmS8, p->s_r2o);
        d.m_CellToInputWeights  = weight(p->w_c2i, {U}, DataType::QSymmS16, p->s_c2i);
        d.m_CellToForgetWeights = weight(p->w_c2f, {U}, DataType::QSymmS16, p->s_c2f);
        d.m_CellToOutputWeights = weight(p->w_c2o, {U}, DataType::QSymmS16, p->s_c2o);
        d.m_InputGateBias  = weight(p->b_i, {U}, DataType::Signed32, p->s_bi);
        d.m_ForgetGateBias = weight(p->b_f, {U}, DataType::Signed32, p->s_bf);
        d.m_CellBias       = weight(p->b_c, {U}, DataType::Signed32, p->s_bc);
        d.m_OutputGateBias = weight(p->b_o, {U}, DataType::Signed32, p->s_bo);
        d.m_InputLayerNormWeights  = weight(p->ln_i, {U}, DataType::QSymmS16, p->s_lni);
        d.m_ForgetLayerNormWeights = weight(p->ln_f, {U}, DataType::QSymmS16, p->s_lnf);
        d.m_CellLayerNormWeights   = weight(p->ln_c, {U}, DataType::QSymmS16, p->s_lnc);
        d.m_OutputLayerNormWeights = weight(p->ln_o, {U}, DataType::QSymmS16, p->s_lno);
        d.m_ProjectionWeights = weight(p->w_proj, {O, U}, DataType::QSymmS8, p->s_proj);
        d.m_ProjectionBias    = weight(p->b_proj, {O}, DataType::Signed32, p->s_bproj);

        h.in(d, xi, p->input);
        h.in(d, hi, p->output_state_in);
        h.in(d, ci, p->cell_state_in);
        auto* o0 = h.out(d, hi);
        auto* o1 = h.out(d, ci);
        auto* o2 = h.out(d, oi);
        h.run(LayerType::QLstm, d);
        copy_out(o0, p->output_state_out, hi.GetNumBytes());
        copy_out(o1, p->cell_state_out, ci.GetNumBytes());
        copy_out(o2, p->output, oi.GetNumBytes());
    });
}

// ================================================================================================
// Part 2: graph-level binding
// ================================================================================================

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
                      int pad_right, int dil_h, int dil_w, int bias_enabled)
{
    auto* n = static_cast<CNet*>(vn);
    if (depthwise) {
        DepthwiseConvolution2dDescriptor d;
        d.m_StrideX = stride_w; d.m_StrideY = stride_h; d.m_PadTop = pad_top; d.m_PadBottom = pad_bottom;
        d.m_PadLeft = pad_left; d.m_PadRight = pad_right; d.m_DilationX = dil_w; d.m_DilationY = dil_h;
        d.m_BiasEnabled = bias_enabled != 0; d.m_DataLayout = DataLayout::NHWC;
        return add_layer(n, n->net->AddDepthwiseConvolution2dLayer(d));
    }
    Convolution2dDescriptor d;
    d.m_StrideX = stride_w; d.m_StrideY = stride_h; d.m_PadTop = pad_top; d.m_PadBottom = pad_bottom;
    d.m_PadLeft = pad_left; d.m_PadRight = pad_right; d.m_DilationX = dil_w; d.m_DilationY = dil_h;
    d.m_BiasEnabled = bias_enabled != 0; d.m_DataLayout = DataLayout::NHWC;
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
                      int pad_top, int pad_bottom, int pad_left, int pad_right)
{
    auto* n = static_cast<CNet*>(vn);
    Pooling2dDescriptor d;
    d.m_PoolType = static_cast<PoolingAlgorithm>(pool_type); d.m_PaddingMethod = static_cast<PaddingMethod>(padding_method);
    d.m_PoolHeight = pool_h; d.m_PoolWidth = pool_w; d.m_StrideX = stride_w; d.m_StrideY = stride_h;
    d.m_PadTop = pad_top; d.m_PadBottom = pad_bottom; d.m_PadLeft = pad_left; d.m_PadRight = pad_right;
    d.m_OutputShapeRounding = OutputShapeRounding::Floor; d.m_DataLayout = DataLayout::NHWC;
    return add_layer(n, n->net->AddPooling2dLayer(d));
}

int armnnc_add_elementwise_binary(void* vn, int op)
{
    auto* n = static_cast<CNet*>(vn);
    return add_layer(n, n->net->AddElementwiseBinaryLayer(ElementwiseBinaryDescriptor(static_cast<BinaryOperation>(op))));
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
