// TEST INFRASTRUCTURE ONLY — a C binding over the CpuRef workloads of the unmodified Arm NN reference
// (oracle/_ref/libarmnn.so), so that Python tests can run the *real* CpuRef workload of a single layer.
//
// Workload-level execution, the way the reference's own layer tests drive a backend
// (src/backends/backendsCommon/test/layerTests/Conv2dTestImpl.cpp:3562-3669): build TensorInfos and a
// QueueDescriptor by hand, RefWorkloadFactory::CreateWorkload, Execute.  The functions take the same
// parameter structs as include/b200k.h, with HOST pointers, so a test hands one struct to the CPU
// restatement, to real CpuRef and (with device pointers) to the CUDA library.
//
// (Whole graphs — INetwork -> Optimize -> LoadNetwork -> EnqueueWorkload on CpuRef or B200Acc — go through the
// runtime binding armnn_b200/host/armnn_capi.cpp.)
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
#include "move_desc.h"

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

extern "C" int cpuref_conv2d_f32(const b200k_conv2d_params* p)   { return cpuref_conv2d_q8(p, 0, 0, 0.f, 0.f); }
extern "C" int cpuref_dwconv2d_f32(const b200k_conv2d_params* p) { return cpuref_conv2d_q8(p, 1, 0, 0.f, 0.f); }
extern "C" int cpuref_fully_connected_q8(const b200k_fc_params* p, int act_kind, float act_a, float act_b);
extern "C" int cpuref_fully_connected_f32(const b200k_fc_params* p) { return cpuref_fully_connected_q8(p, 0, 0.f, 0.f); }

extern "C" int cpuref_transpose_conv2d_q8(const b200k_conv2d_params* p)
{
    return guarded([&] {
        Harness h;
        const unsigned N = p->n, H = p->h, W = p->wd, C = p->c, OH = p->oh, OW = p->ow, OC = p->oc, KH = p->kh, KW = p->kw;
        TensorInfo xi = make_info(p->x, TensorShape({N, H, W, C}), 0, 0, false);
        TensorInfo wi = make_info(p->w, TensorShape({OC, KH, KW, C}), 0, OC, true);
        TensorInfo yi = make_info(p->y, TensorShape({N, OH, OW, OC}), 0, 0, false);
        TransposeConvolution2dQueueDescriptor d;
        d.m_Parameters.m_PadTop = p->pad_top; d.m_Parameters.m_PadLeft = p->pad_left;
        d.m_Parameters.m_PadBottom = 0; d.m_Parameters.m_PadRight = 0;
        d.m_Parameters.m_StrideX = p->stride_w; d.m_Parameters.m_StrideY = p->stride_h;
        d.m_Parameters.m_BiasEnabled = p->bias.data != nullptr;
        d.m_Parameters.m_DataLayout = DataLayout::NHWC;
        ScopedTensorHandle weights(wi), bias(p->bias.data ? make_info(p->bias, TensorShape({OC}), 0, OC, true) : TensorInfo({1}, DataType::Signed32));
        weights.Allocate(); bias.Allocate();
        std::memcpy(weights.GetTensor<void>(), p->w.data, wi.GetNumBytes());
        d.m_Weight = &weights;
        if (p->bias.data) {
            std::memcpy(bias.GetTensor<void>(), p->bias.data, OC * sizeof(int32_t));
            d.m_Bias = &bias;
        }
        h.in(d, xi, p->x.data);
        ITensorHandle* o = h.out(d, yi);
        h.run(LayerType::TransposeConvolution2d, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
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

extern "C" int cpuref_batch_matmul_f32(const b200k_bmm_params* p) { return cpuref_batch_matmul_q8(p); }

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
        if (p->op >= 200)
        {
            // Comparison (any input type) and LogicalBinary (Boolean inputs): Boolean output, one byte per element
            oi = TensorInfo(shape(p->shape_out), DataType::Boolean);
            if (p->op >= 210)
            {
                ai = TensorInfo(shape(p->shape_a), DataType::Boolean);
                bi = TensorInfo(shape(p->shape_b), DataType::Boolean);
                LogicalBinaryQueueDescriptor d;
                d.m_Parameters.m_Operation = p->op == 210 ? LogicalBinaryOperation::LogicalAnd : LogicalBinaryOperation::LogicalOr;
                h.in(d, ai, p->a.data);
                h.in(d, bi, p->b.data);
                auto* o = h.out(d, oi);
                h.run(LayerType::LogicalBinary, d);
                copy_out(o, const_cast<void*>(p->out.data), oi.GetNumBytes());
            }
            else
            {
                ComparisonQueueDescriptor d;
                d.m_Parameters.m_Operation = static_cast<ComparisonOperation>(p->op - 200);
                h.in(d, ai, p->a.data);
                h.in(d, bi, p->b.data);
                auto* o = h.out(d, oi);
                h.run(LayerType::Comparison, d);
                copy_out(o, const_cast<void*>(p->out.data), oi.GetNumBytes());
            }
            return;
        }
        if (p->op == B200K_ELTWISE_PRELU)
        {
            PreluQueueDescriptor d;
            h.in(d, ai, p->a.data);
            h.in(d, bi, p->b.data);
            auto* o = h.out(d, oi);
            h.run(LayerType::Prelu, d);
            copy_out(o, const_cast<void*>(p->out.data), oi.GetNumBytes());
        }
        else
        {
            ElementwiseBinaryQueueDescriptor d;
            d.m_Parameters.m_Operation = static_cast<BinaryOperation>(p->op);
            h.in(d, ai, p->a.data);
            h.in(d, bi, p->b.data);
            auto* o = h.out(d, oi);
            h.run(LayerType::ElementwiseBinary, d);
            copy_out(o, const_cast<void*>(p->out.data), oi.GetNumBytes());
        }
        run_activation(act_kind, act_a, act_b, oi, const_cast<void*>(p->out.data));
    });
}

extern "C" int cpuref_activation_q8(const b200k_activation_params* p)
{
    return guarded([&] {
        Harness h;
        TensorInfo xi = make_info(p->x, TensorShape({(unsigned)p->count}), 0, 0, false);
        TensorInfo yi = make_info(p->y, TensorShape({(unsigned)p->count}), 0, 0, false);
        if (p->function == B200K_ACTIVATION_FAKE_QUANTIZATION)
        {
            FakeQuantizationQueueDescriptor fq;
            fq.m_Parameters.m_Min = p->a; fq.m_Parameters.m_Max = p->b;
            // the queue descriptor's Validate wants two dimensions
            TensorInfo x2 = make_info(p->x, TensorShape({1u, (unsigned)p->count}), 0, 0, false);
            TensorInfo y2 = make_info(p->y, TensorShape({1u, (unsigned)p->count}), 0, 0, false);
            h.in(fq, x2, p->x.data);
            auto* fo = h.out(fq, y2);
            h.run(LayerType::FakeQuantization, fq);
            copy_out(fo, const_cast<void*>(p->y.data), yi.GetNumBytes());
            return;
        }
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

extern "C" int cpuref_gather_q(const b200k_gather_params* p)
{
    return guarded([&] {
        Harness h;
        TensorInfo xi = make_info(p->x, TensorShape({(unsigned)p->outer, (unsigned)p->axis_size, (unsigned)p->inner}), 0, 0, false);
        TensorInfo ii(TensorShape({(unsigned)p->n_indices}), DataType::Signed32);
        TensorInfo yi = make_info(p->y, TensorShape({(unsigned)p->outer, (unsigned)p->n_indices, (unsigned)p->inner}), 0, 0, false);
        GatherQueueDescriptor d;
        d.m_Parameters.m_Axis = 1;
        h.in(d, xi, p->x.data);
        h.in(d, ii, p->indices);
        auto* o = h.out(d, yi);
        h.run(LayerType::Gather, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_reverse_q(const b200k_reverse_params* p)
{
    return guarded([&] {
        Harness h;
        unsigned dims[6];
        for (int d = 0; d < p->rank; ++d) dims[d] = (unsigned)p->shape[d];
        TensorInfo xi = make_info(p->x, TensorShape((unsigned)p->rank, dims), 0, 0, false);
        TensorInfo ai(TensorShape({(unsigned)p->n_axes}), DataType::Signed32);
        TensorInfo yi = make_info(p->y, TensorShape((unsigned)p->rank, dims), 0, 0, false);
        ReverseV2QueueDescriptor d;
        h.in(d, xi, p->x.data);
        h.in(d, ai, p->axes);
        auto* o = h.out(d, yi);
        h.run(LayerType::ReverseV2, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_gather_nd_q(const b200k_gather_nd_params* p)
{
    return guarded([&] {
        Harness h;
        unsigned dims[6];
        for (int d = 0; d < p->nd; ++d) dims[d] = (unsigned)p->dims[d];
        dims[p->nd] = (unsigned)p->inner;
        TensorInfo xi = make_info(p->x, TensorShape((unsigned)p->nd + 1, dims), 0, 0, false);
        TensorInfo ii(TensorShape({(unsigned)p->n_indices, (unsigned)p->nd}), DataType::Signed32);
        TensorInfo yi = make_info(p->y, TensorShape({(unsigned)p->n_indices, (unsigned)p->inner}), 0, 0, false);
        GatherNdQueueDescriptor d;
        h.in(d, xi, p->x.data);
        h.in(d, ii, p->indices);
        auto* o = h.out(d, yi);
        h.run(LayerType::GatherNd, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_batch_norm_q(const b200k_batch_norm_params* p)
{
    return guarded([&] {
        Harness h;
        TensorShape s = p->nchw ? TensorShape({(unsigned)p->n, (unsigned)p->c, 1u, (unsigned)p->hw})
                                : TensorShape({(unsigned)p->n, 1u, (unsigned)p->hw, (unsigned)p->c});
        TensorInfo xi = make_info(p->x, s, 0, 0, false);
        TensorInfo yi = make_info(p->y, s, 0, 0, false);
        BatchNormalizationQueueDescriptor d;
        d.m_Parameters.m_Eps = p->eps;
        d.m_Parameters.m_DataLayout = p->nchw ? DataLayout::NCHW : DataLayout::NHWC;
        TensorShape cs({(unsigned)p->c});
        auto constant = [&](const b200k_qtensor& t) {
            TensorInfo ti = make_info(t, cs, 0, 0, true);
            auto handle = std::make_unique<ScopedTensorHandle>(ti);
            handle->Allocate();
            std::memcpy(handle->GetTensor<void>(), t.data, ti.GetNumBytes());
            return handle;
        };
        auto mean = constant(p->mean), var = constant(p->variance), beta = constant(p->beta), gamma = constant(p->gamma);
        d.m_Mean = mean.get(); d.m_Variance = var.get(); d.m_Beta = beta.get(); d.m_Gamma = gamma.get();
        h.in(d, xi, p->x.data);
        auto* o = h.out(d, yi);
        h.run(LayerType::BatchNormalization, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_instance_norm_q(const b200k_instance_norm_params* p)
{
    return guarded([&] {
        Harness h;
        TensorShape s = p->nchw ? TensorShape({(unsigned)p->n, (unsigned)p->c, 1u, (unsigned)p->hw})
                                : TensorShape({(unsigned)p->n, 1u, (unsigned)p->hw, (unsigned)p->c});
        TensorInfo xi = make_info(p->x, s, 0, 0, false);
        TensorInfo yi = make_info(p->y, s, 0, 0, false);
        InstanceNormalizationQueueDescriptor d;
        d.m_Parameters.m_Gamma = p->gamma; d.m_Parameters.m_Beta = p->beta; d.m_Parameters.m_Eps = p->eps;
        d.m_Parameters.m_DataLayout = p->nchw ? DataLayout::NCHW : DataLayout::NHWC;
        h.in(d, xi, p->x.data);
        auto* o = h.out(d, yi);
        h.run(LayerType::InstanceNormalization, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_normalization_q(const b200k_normalization_params* p)
{
    return guarded([&] {
        Harness h;
        TensorShape s = p->nchw ? TensorShape({(unsigned)p->n, (unsigned)p->c, (unsigned)p->h, (unsigned)p->w})
                                : TensorShape({(unsigned)p->n, (unsigned)p->h, (unsigned)p->w, (unsigned)p->c});
        TensorInfo xi = make_info(p->x, s, 0, 0, false);
        TensorInfo yi = make_info(p->y, s, 0, 0, false);
        NormalizationQueueDescriptor d;
        d.m_Parameters.m_NormChannelType = p->channel_type ? NormalizationAlgorithmChannel::Within : NormalizationAlgorithmChannel::Across;
        d.m_Parameters.m_NormMethodType = NormalizationAlgorithmMethod::LocalBrightness;
        d.m_Parameters.m_NormSize = p->norm_size;
        d.m_Parameters.m_Alpha = p->alpha; d.m_Parameters.m_Beta = p->beta; d.m_Parameters.m_K = p->kappa;
        d.m_Parameters.m_DataLayout = p->nchw ? DataLayout::NCHW : DataLayout::NHWC;
        h.in(d, xi, p->x.data);
        auto* o = h.out(d, yi);
        h.run(LayerType::Normalization, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_cast_q(const b200k_convert_params* p)
{
    return guarded([&] {
        Harness h;
        const TensorShape shape({(unsigned)p->count});
        TensorInfo xi = make_info(p->x, shape, 0, 0, false), yi = make_info(p->y, shape, 0, 0, false);
        CastQueueDescriptor d;
        h.in(d, xi, p->x.data);
        ITensorHandle* o = h.out(d, yi);
        h.run(LayerType::Cast, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_conv3d_q(const b200k_conv3d_params* p)
{
    return guarded([&] {
        Harness h;
        const unsigned OC = (unsigned)p->oc;
        TensorInfo xi = make_info(p->x, TensorShape({(unsigned)p->n, (unsigned)p->d, (unsigned)p->h, (unsigned)p->wd, (unsigned)p->c}), 0, 0, false);
        TensorInfo wi = make_info(p->w, TensorShape({(unsigned)p->kd, (unsigned)p->kh, (unsigned)p->kw, (unsigned)p->c, OC}), 4, OC, true);
        TensorInfo yi = make_info(p->y, TensorShape({(unsigned)p->n, (unsigned)p->od, (unsigned)p->oh, (unsigned)p->ow, OC}), 0, 0, false);
        Convolution3dQueueDescriptor d;
        auto& q = d.m_Parameters;
        q.m_PadFront = (unsigned)p->pad_front; q.m_PadTop = (unsigned)p->pad_top; q.m_PadLeft = (unsigned)p->pad_left;
        q.m_PadBack = 0; q.m_PadBottom = 0; q.m_PadRight = 0;          // only shape inference reads them
        q.m_StrideX = (unsigned)p->stride_w; q.m_StrideY = (unsigned)p->stride_h; q.m_StrideZ = (unsigned)p->stride_d;
        q.m_DilationX = (unsigned)p->dil_w; q.m_DilationY = (unsigned)p->dil_h; q.m_DilationZ = (unsigned)p->dil_d;
        q.m_BiasEnabled = p->bias.data != nullptr;
        q.m_DataLayout = DataLayout::NDHWC;
        h.in(d, xi, p->x.data);
        h.in(d, wi, p->w.data);
        if (p->bias.data) h.in(d, make_info(p->bias, TensorShape({OC}), 0, OC, true), p->bias.data);
        ITensorHandle* o = h.out(d, yi);
        h.run(LayerType::Convolution3d, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_pool3d_q(const b200k_pool3d_params* p)
{
    return guarded([&] {
        Harness h;
        TensorInfo xi = make_info(p->x, TensorShape({(unsigned)p->n, (unsigned)p->d, (unsigned)p->h, (unsigned)p->wd, (unsigned)p->c}), 0, 0, false);
        TensorInfo yi = make_info(p->y, TensorShape({(unsigned)p->n, (unsigned)p->od, (unsigned)p->oh, (unsigned)p->ow, (unsigned)p->c}), 0, 0, false);
        Pooling3dQueueDescriptor d;
        auto& q = d.m_Parameters;
        q.m_PoolType = static_cast<PoolingAlgorithm>(p->pool_type);
        q.m_PaddingMethod = p->padding_method == 1 ? PaddingMethod::Exclude : PaddingMethod::IgnoreValue;
        q.m_PoolDepth = (unsigned)p->pool_d; q.m_PoolHeight = (unsigned)p->pool_h; q.m_PoolWidth = (unsigned)p->pool_w;
        q.m_StrideZ = (unsigned)p->stride_d; q.m_StrideY = (unsigned)p->stride_h; q.m_StrideX = (unsigned)p->stride_w;
        q.m_PadFront = (unsigned)p->pad_front; q.m_PadBack = (unsigned)p->pad_back; q.m_PadTop = (unsigned)p->pad_top;
        q.m_PadBottom = (unsigned)p->pad_bottom; q.m_PadLeft = (unsigned)p->pad_left; q.m_PadRight = (unsigned)p->pad_right;
        q.m_OutputShapeRounding = OutputShapeRounding::Floor;
        q.m_DataLayout = DataLayout::NDHWC;
        h.in(d, xi, p->x.data);
        ITensorHandle* o = h.out(d, yi);
        h.run(LayerType::Pooling3d, d);
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

extern "C" int cpuref_log_softmax_q(const b200k_softmax_params* p)
{
    return guarded([&] {
        Harness h;
        TensorShape s({(unsigned)p->outer, (unsigned)p->axis_size, (unsigned)p->inner});
        TensorInfo xi = make_info(p->x, s, 0, 0, false);
        TensorInfo yi = make_info(p->y, s, 0, 0, false);
        LogSoftmaxQueueDescriptor d;
        d.m_Parameters.m_Beta = p->beta;
        d.m_Parameters.m_Axis = 1;
        h.in(d, xi, p->x.data);
        auto* o = h.out(d, yi);
        h.run(LayerType::LogSoftmax, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_l2_normalization_q(const b200k_softmax_params* p)
{
    return guarded([&] {
        Harness h;
        // the channel axis is the row axis: NHWC [outer, 1, 1, axis] when it is contiguous, else NCHW [outer, axis, 1, inner]
        const bool nhwc = p->inner == 1;
        TensorShape s = nhwc ? TensorShape({(unsigned)p->outer, 1u, 1u, (unsigned)p->axis_size})
                             : TensorShape({(unsigned)p->outer, (unsigned)p->axis_size, 1u, (unsigned)p->inner});
        TensorInfo xi = make_info(p->x, s, 0, 0, false);
        TensorInfo yi = make_info(p->y, s, 0, 0, false);
        L2NormalizationQueueDescriptor d;
        d.m_Parameters.m_Eps = p->beta;
        d.m_Parameters.m_DataLayout = nhwc ? DataLayout::NHWC : DataLayout::NCHW;
        h.in(d, xi, p->x.data);
        auto* o = h.out(d, yi);
        h.run(LayerType::L2Normalization, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_arg_min_max_q(const b200k_arg_min_max_params* p)
{
    return guarded([&] {
        Harness h;
        TensorInfo xi = make_info(p->x, TensorShape({(unsigned)p->outer, (unsigned)p->axis_size, (unsigned)p->inner}), 0, 0, false);
        TensorInfo yi(TensorShape({(unsigned)p->outer, (unsigned)p->inner}), p->out_int64 ? DataType::Signed64 : DataType::Signed32);
        ArgMinMaxQueueDescriptor d;
        d.m_Parameters.m_Function = p->function ? ArgMinMaxFunction::Max : ArgMinMaxFunction::Min;
        d.m_Parameters.m_Axis = 1;
        h.in(d, xi, p->x.data);
        auto* o = h.out(d, yi);
        h.run(LayerType::ArgMinMax, d);
        copy_out(o, p->y, yi.GetNumBytes());
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

extern "C" int cpuref_pad_q(const b200k_pad_params* p)
{
    return guarded([&] {
        Harness h;
        unsigned in_dims[4], out_dims[4];
        PadQueueDescriptor d;
        for (int i = 0; i < p->rank; ++i) {
            in_dims[i] = (unsigned)p->shape[i];
            out_dims[i] = (unsigned)(p->shape[i] + p->pad_before[i] + p->pad_after[i]);
            d.m_Parameters.m_PadList.emplace_back((unsigned)p->pad_before[i], (unsigned)p->pad_after[i]);
        }
        d.m_Parameters.m_PadValue = p->pad_value;
        d.m_Parameters.m_PaddingMode = p->mode == 1 ? PaddingMode::Reflect : p->mode == 2 ? PaddingMode::Symmetric : PaddingMode::Constant;
        TensorInfo xi = make_info(p->x, TensorShape((unsigned)p->rank, in_dims), 0, 0, false);
        TensorInfo yi = make_info(p->y, TensorShape((unsigned)p->rank, out_dims), 0, 0, false);
        h.in(d, xi, p->x.data);
        ITensorHandle* o = h.out(d, yi);
        h.run(LayerType::Pad, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_unary_q(const b200k_unary_params* p)
{
    return guarded([&] {
        Harness h;
        const TensorShape shape({(unsigned)p->count});
        TensorInfo xi = make_info(p->x, shape, 0, 0, false), yi = make_info(p->y, shape, 0, 0, false);
        if (p->operation == 5)                     // LogicalNot: Boolean tensors
        {
            TensorInfo bx(shape, DataType::Boolean), by(shape, DataType::Boolean);
            ElementwiseUnaryQueueDescriptor ld;
            ld.m_Parameters.m_Operation = UnaryOperation::LogicalNot;
            h.in(ld, bx, p->x.data);
            ITensorHandle* lo = h.out(ld, by);
            h.run(LayerType::ElementwiseUnary, ld);
            copy_out(lo, const_cast<void*>(p->y.data), by.GetNumBytes());
            return;
        }
        if (p->operation == 9)                     // the Floor layer
        {
            FloorQueueDescriptor fd;
            h.in(fd, xi, p->x.data);
            ITensorHandle* fo = h.out(fd, yi);
            h.run(LayerType::Floor, fd);
            copy_out(fo, const_cast<void*>(p->y.data), yi.GetNumBytes());
            return;
        }
        ElementwiseUnaryQueueDescriptor d;
        d.m_Parameters.m_Operation = static_cast<UnaryOperation>(p->operation);
        h.in(d, xi, p->x.data);
        ITensorHandle* o = h.out(d, yi);
        h.run(LayerType::ElementwiseUnary, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_reduce_q(const b200k_reduce_params* p)
{
    return guarded([&] {
        Harness h;
        ReduceQueueDescriptor d;
        d.m_Parameters.m_KeepDims = false;
        d.m_Parameters.m_ReduceOperation = static_cast<ReduceOperation>(p->op);
        unsigned in_dims[6], out_dims[6], nout = 0;
        for (int i = 0; i < p->rank; ++i) {
            in_dims[i] = (unsigned)p->shape[i];
            if (p->axis_mask & (1 << i)) d.m_Parameters.m_vAxis.push_back((uint32_t)i);
            else if (p->axis_mask) out_dims[nout++] = (unsigned)p->shape[i];
        }
        if (nout == 0) out_dims[nout++] = 1;
        TensorInfo xi = make_info(p->x, TensorShape((unsigned)p->rank, in_dims), 0, 0, false);
        TensorInfo yi = make_info(p->y, TensorShape(nout, out_dims), 0, 0, false);
        h.in(d, xi, p->x.data);
        ITensorHandle* o = h.out(d, yi);
        h.run(LayerType::Reduce, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

extern "C" int cpuref_resize_q(const b200k_resize_params* p)
{
    return guarded([&] {
        Harness h;
        ResizeQueueDescriptor d;
        d.m_Parameters.m_TargetHeight = (uint32_t)p->out_h;
        d.m_Parameters.m_TargetWidth = (uint32_t)p->out_w;
        d.m_Parameters.m_Method = p->method == 0 ? ResizeMethod::Bilinear : ResizeMethod::NearestNeighbor;
        d.m_Parameters.m_DataLayout = p->nchw ? DataLayout::NCHW : DataLayout::NHWC;
        d.m_Parameters.m_AlignCorners = p->align_corners != 0;
        d.m_Parameters.m_HalfPixelCenters = p->half_pixel_centers != 0;
        const unsigned N = (unsigned)p->n, C = (unsigned)p->c;
        const TensorShape xs = p->nchw ? TensorShape({N, C, (unsigned)p->in_h, (unsigned)p->in_w}) : TensorShape({N, (unsigned)p->in_h, (unsigned)p->in_w, C});
        const TensorShape ys = p->nchw ? TensorShape({N, C, (unsigned)p->out_h, (unsigned)p->out_w}) : TensorShape({N, (unsigned)p->out_h, (unsigned)p->out_w, C});
        TensorInfo xi = make_info(p->x, xs, 0, 0, false), yi = make_info(p->y, ys, 0, 0, false);
        h.in(d, xi, p->x.data);
        ITensorHandle* o = h.out(d, yi);
        h.run(LayerType::Resize, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}

// Concat, Splitter, Permute, Transpose, StridedSlice, Slice: the real RefConcatWorkload ... RefSliceWorkload on the
// descriptor the test states (oracle/move_desc.h).
extern "C" int cpuref_move_q(const oracle_move_params* p)
{
    return guarded([&] {
        Harness h;
        const unsigned rank = (unsigned)p->rank;
        auto shape_of = [&](const int32_t* s, unsigned r) {
            unsigned dims[6];
            for (unsigned i = 0; i < r; ++i) dims[i] = (unsigned)s[i];
            return TensorShape(r, dims);
        };
        const TensorInfo whole = make_info(p->whole, shape_of(p->whole_shape, rank), 0, 0, false);
        std::vector<TensorInfo> views;
        for (int v = 0; v < p->n_views; ++v)
            views.push_back(make_info(p->view[v], shape_of(p->view_shape[v], p->view_rank[v] ? (unsigned)p->view_rank[v] : rank), 0, 0, false));
        std::vector<ITensorHandle*> outs;
        switch (p->kind) {
            case MOVE_CONCAT: {
                ConcatQueueDescriptor d;
                d.m_Parameters = OriginsDescriptor((uint32_t)p->n_views, rank);
                for (int v = 0; v < p->n_views; ++v) {
                    std::vector<unsigned> origin(p->view_origin[v], p->view_origin[v] + rank);
                    for (unsigned i = 0; i < rank; ++i) d.m_Parameters.SetViewOriginCoord((uint32_t)v, i, origin[i]);
                    d.m_ViewOrigins.emplace_back(origin);
                    h.in(d, views[(size_t)v], p->view[v].data);
                }
                ITensorHandle* o = h.out(d, whole);
                std::memcpy(o->Map(), p->whole.data, whole.GetNumBytes());      // (elements no view covers keep their value)
                o->Unmap();
                h.run(LayerType::Concat, d);
                copy_out(o, const_cast<void*>(p->whole.data), whole.GetNumBytes());
                break;
            }
            case MOVE_SPLIT: {
                SplitterQueueDescriptor d;
                d.m_Parameters = ViewsDescriptor((uint32_t)p->n_views, rank);
                h.in(d, whole, p->whole.data);
                for (int v = 0; v < p->n_views; ++v) {
                    std::vector<unsigned> origin(p->view_origin[v], p->view_origin[v] + rank);
                    for (unsigned i = 0; i < rank; ++i) {
                        d.m_Parameters.SetViewOriginCoord((uint32_t)v, i, origin[i]);
                        d.m_Parameters.SetViewSize((uint32_t)v, i, (uint32_t)p->view_shape[v][i]);
                    }
                    d.m_ViewOrigins.emplace_back(origin);
                    outs.push_back(h.out(d, views[(size_t)v]));
                }
                h.run(LayerType::Splitter, d);
                for (int v = 0; v < p->n_views; ++v) copy_out(outs[(size_t)v], const_cast<void*>(p->view[v].data), views[(size_t)v].GetNumBytes());
                break;
            }
            case MOVE_PERMUTE:
            case MOVE_TRANSPOSE: {
                unsigned m[6];
                for (unsigned i = 0; i < rank; ++i) m[i] = (unsigned)p->perm[i];
                const PermutationVector pv(m, rank);
                if (p->kind == MOVE_PERMUTE) {
                    PermuteQueueDescriptor d;
                    d.m_Parameters = PermuteDescriptor(pv);
                    h.in(d, whole, p->whole.data);
                    outs.push_back(h.out(d, views[0]));
                    h.run(LayerType::Permute, d);
                } else {
                    TransposeQueueDescriptor d;
                    d.m_Parameters = TransposeDescriptor(pv);
                    h.in(d, whole, p->whole.data);
                    outs.push_back(h.out(d, views[0]));
                    h.run(LayerType::Transpose, d);
                }
                copy_out(outs[0], const_cast<void*>(p->view[0].data), views[0].GetNumBytes());
                break;
            }
            case MOVE_STRIDED_SLICE: {
                StridedSliceQueueDescriptor d;
                d.m_Parameters.m_Begin.assign(p->begin, p->begin + rank);
                d.m_Parameters.m_End.assign(p->end, p->end + rank);
                d.m_Parameters.m_Stride.assign(p->stride, p->stride + rank);
                d.m_Parameters.m_BeginMask = p->begin_mask;
                d.m_Parameters.m_EndMask = p->end_mask;
                d.m_Parameters.m_ShrinkAxisMask = p->shrink_axis_mask;
                h.in(d, whole, p->whole.data);
                outs.push_back(h.out(d, views[0]));
                h.run(LayerType::StridedSlice, d);
                copy_out(outs[0], const_cast<void*>(p->view[0].data), views[0].GetNumBytes());
                break;
            }
            case MOVE_SLICE: {
                SliceQueueDescriptor d;
                d.m_Parameters.m_Begin.assign(p->begin, p->begin + rank);
                d.m_Parameters.m_Size.assign(p->end, p->end + rank);
                h.in(d, whole, p->whole.data);
                outs.push_back(h.out(d, views[0]));
                h.run(LayerType::Slice, d);
                copy_out(outs[0], const_cast<void*>(p->view[0].data), views[0].GetNumBytes());
                break;
            }
            case MOVE_DEPTH_TO_SPACE: {
                DepthToSpaceQueueDescriptor d;
                d.m_Parameters.m_BlockSize = (unsigned)p->perm[0];
                d.m_Parameters.m_DataLayout = p->perm[1] ? DataLayout::NCHW : DataLayout::NHWC;
                h.in(d, whole, p->whole.data);
                outs.push_back(h.out(d, views[0]));
                h.run(LayerType::DepthToSpace, d);
                copy_out(outs[0], const_cast<void*>(p->view[0].data), views[0].GetNumBytes());
                break;
            }
            case MOVE_SPACE_TO_DEPTH: {
                SpaceToDepthQueueDescriptor d;
                d.m_Parameters.m_BlockSize = (unsigned)p->perm[0];
                d.m_Parameters.m_DataLayout = p->perm[1] ? DataLayout::NCHW : DataLayout::NHWC;
                h.in(d, whole, p->whole.data);
                outs.push_back(h.out(d, views[0]));
                h.run(LayerType::SpaceToDepth, d);
                copy_out(outs[0], const_cast<void*>(p->view[0].data), views[0].GetNumBytes());
                break;
            }
            case MOVE_CHANNEL_SHUFFLE: {
                ChannelShuffleQueueDescriptor d;
                d.m_Parameters.m_Axis = (uint32_t)p->perm[0];
                d.m_Parameters.m_NumGroups = (uint32_t)p->perm[1];
                h.in(d, whole, p->whole.data);
                outs.push_back(h.out(d, views[0]));
                h.run(LayerType::ChannelShuffle, d);
                copy_out(outs[0], const_cast<void*>(p->view[0].data), views[0].GetNumBytes());
                break;
            }
            case MOVE_BATCH_TO_SPACE: {
                BatchToSpaceNdQueueDescriptor d;
                const unsigned sp = (unsigned)p->rank - 2;
                d.m_Parameters.m_DataLayout = p->perm[0] ? DataLayout::NCHW : DataLayout::NHWC;
                d.m_Parameters.m_BlockShape.clear(); d.m_Parameters.m_Crops.clear();
                for (unsigned i = 0; i < sp; ++i)
                {
                    d.m_Parameters.m_BlockShape.push_back((unsigned)p->begin[i]);
                    d.m_Parameters.m_Crops.emplace_back((unsigned)p->end[i], (unsigned)p->stride[i]);
                }
                h.in(d, whole, p->whole.data);
                outs.push_back(h.out(d, views[0]));
                h.run(LayerType::BatchToSpaceNd, d);
                copy_out(outs[0], const_cast<void*>(p->view[0].data), views[0].GetNumBytes());
                break;
            }
            case MOVE_SPACE_TO_BATCH: {
                SpaceToBatchNdQueueDescriptor d;
                const unsigned sp = (unsigned)p->rank - 2;
                d.m_Parameters.m_DataLayout = p->perm[0] ? DataLayout::NCHW : DataLayout::NHWC;
                d.m_Parameters.m_BlockShape.clear(); d.m_Parameters.m_PadList.clear();
                for (unsigned i = 0; i < sp; ++i)
                {
                    d.m_Parameters.m_BlockShape.push_back((unsigned)p->begin[i]);
                    d.m_Parameters.m_PadList.emplace_back((unsigned)p->end[i], (unsigned)p->stride[i]);
                }
                h.in(d, whole, p->whole.data);
                outs.push_back(h.out(d, views[0]));
                h.run(LayerType::SpaceToBatchNd, d);
                copy_out(outs[0], const_cast<void*>(p->view[0].data), views[0].GetNumBytes());
                break;
            }
            case MOVE_TILE: {
                TileQueueDescriptor d;
                d.m_Parameters.m_Multiples.clear();
                for (int i = 0; i < p->rank; ++i) d.m_Parameters.m_Multiples.push_back((uint32_t)p->perm[i]);
                h.in(d, whole, p->whole.data);
                outs.push_back(h.out(d, views[0]));
                h.run(LayerType::Tile, d);
                copy_out(outs[0], const_cast<void*>(p->view[0].data), views[0].GetNumBytes());
                break;
            }
            case MOVE_BROADCAST_TO: {
                BroadcastToQueueDescriptor d;
                d.m_Parameters.m_BroadcastToShape = views[0].GetShape();
                h.in(d, whole, p->whole.data);
                outs.push_back(h.out(d, views[0]));
                h.run(LayerType::BroadcastTo, d);
                copy_out(outs[0], const_cast<void*>(p->view[0].data), views[0].GetNumBytes());
                break;
            }
            case MOVE_STACK: {
                StackQueueDescriptor d;
                d.m_Parameters.m_Axis = (uint32_t)p->perm[0];
                d.m_Parameters.m_NumInputs = (uint32_t)p->n_views;
                d.m_Parameters.m_InputShape = views[0].GetShape();
                for (int v = 0; v < p->n_views; ++v) h.in(d, views[(size_t)v], p->view[v].data);
                ITensorHandle* o = h.out(d, whole);
                h.run(LayerType::Stack, d);
                copy_out(o, const_cast<void*>(p->whole.data), whole.GetNumBytes());
                break;
            }
            default: throw InvalidArgumentException("cpuref_move_q: unknown kind");
        }
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


// The Lstm layer on Float32 tensors (RefLstmWorkload); input_stride / output_stride must be the dense ones here.
extern "C" int cpuref_lstm_step_f32(const b200k_lstm_params* p)
{
    return guarded([&] {
        Harness h;
        const unsigned B = p->batch, I = p->input_size, U = p->num_units, O = p->output_size;
        if (p->input_stride != (int64_t)I || p->output_stride != (int64_t)O) throw InvalidArgumentException("dense rows only");
        TensorInfo xi({B, I}, DataType::Float32), hi({B, O}, DataType::Float32), ci({B, U}, DataType::Float32);
        LstmQueueDescriptor d;
        auto& q = d.m_Parameters;
        q.m_CifgEnabled = p->w_i2i == nullptr;
        q.m_PeepholeEnabled = p->w_c2f != nullptr;
        q.m_ProjectionEnabled = p->w_proj != nullptr;
        q.m_LayerNormEnabled = p->ln_f != nullptr;
        q.m_ActivationFunc = (uint32_t)p->activation;
        q.m_ClippingThresCell = p->cell_clip; q.m_ClippingThresProj = p->projection_clip;
        TensorInfo scratch({B, U * (q.m_CifgEnabled ? 3u : 4u)}, DataType::Float32);
        std::vector<std::unique_ptr<ScopedTensorHandle>> keep;
        auto weight = [&](const float* data, TensorShape shape) -> const ConstTensorHandle* {
            if (!data) return nullptr;
            TensorInfo info(shape, DataType::Float32);
            info.SetConstant(true);
            auto t = std::make_unique<ScopedTensorHandle>(info);
            t->Allocate();
            std::memcpy(t->GetTensor<void>(), data, info.GetNumBytes());
            keep.push_back(std::move(t));
            return keep.back().get();
        };
        d.m_InputToInputWeights  = weight(p->w_i2i, {U, I}); d.m_InputToForgetWeights = weight(p->w_i2f, {U, I});
        d.m_InputToCellWeights   = weight(p->w_i2c, {U, I}); d.m_InputToOutputWeights = weight(p->w_i2o, {U, I});
        d.m_RecurrentToInputWeights  = weight(p->w_r2i, {U, O}); d.m_RecurrentToForgetWeights = weight(p->w_r2f, {U, O});
        d.m_RecurrentToCellWeights   = weight(p->w_r2c, {U, O}); d.m_RecurrentToOutputWeights = weight(p->w_r2o, {U, O});
        d.m_CellToInputWeights = weight(p->w_c2i, {U}); d.m_CellToForgetWeights = weight(p->w_c2f, {U}); d.m_CellToOutputWeights = weight(p->w_c2o, {U});
        d.m_InputGateBias = weight(p->b_i, {U}); d.m_ForgetGateBias = weight(p->b_f, {U});
        d.m_CellBias = weight(p->b_c, {U}); d.m_OutputGateBias = weight(p->b_o, {U});
        d.m_InputLayerNormWeights = weight(p->ln_i, {U}); d.m_ForgetLayerNormWeights = weight(p->ln_f, {U});
        d.m_CellLayerNormWeights = weight(p->ln_c, {U}); d.m_OutputLayerNormWeights = weight(p->ln_o, {U});
        d.m_ProjectionWeights = weight(p->w_proj, {O, U}); d.m_ProjectionBias = weight(p->b_proj, {O});
        h.in(d, xi, p->input);
        h.in(d, hi, p->output_state_in);
        h.in(d, ci, p->cell_state_in);
        h.out(d, scratch);
        auto* o1 = h.out(d, hi);
        auto* o2 = h.out(d, ci);
        auto* o3 = h.out(d, hi);
        h.run(LayerType::Lstm, d);
        copy_out(o1, p->output_state_out, hi.GetNumBytes());
        copy_out(o2, p->cell_state_out, ci.GetNumBytes());
        copy_out(o3, p->output, hi.GetNumBytes());
    });
}

extern "C" int cpuref_convert_fp16(const b200k_convert_fp16_params* p)
{
    return guarded([&] {
        Harness h;
        const TensorShape shape({(unsigned)p->count});
        TensorInfo half(shape, DataType::Float16), single(shape, DataType::Float32);
        if (p->to_half)
        {
            ConvertFp32ToFp16QueueDescriptor d;
            h.in(d, single, p->x);
            ITensorHandle* o = h.out(d, half);
            h.run(LayerType::ConvertFp32ToFp16, d);
            copy_out(o, p->y, half.GetNumBytes());
        }
        else
        {
            ConvertFp16ToFp32QueueDescriptor d;
            h.in(d, half, p->x);
            ITensorHandle* o = h.out(d, single);
            h.run(LayerType::ConvertFp16ToFp32, d);
            copy_out(o, p->y, single.GetNumBytes());
        }
    });
}

extern "C" int cpuref_scatter_nd_q(const b200k_scatter_nd_params* p)
{
    return guarded([&] {
        Harness h;
        unsigned dims[9], udims[9];
        for (int d = 0; d < p->nd; ++d) dims[d] = (unsigned)p->dims[d];
        dims[p->nd] = (unsigned)p->inner;
        udims[0] = (unsigned)p->n_indices; udims[1] = (unsigned)p->inner;
        const TensorShape full((unsigned)p->nd + 1, dims);
        TensorInfo ii(TensorShape({(unsigned)p->n_indices, (unsigned)p->nd}), DataType::Signed32);
        TensorInfo ui = make_info(p->updates, TensorShape(2, udims), 0, 0, false);
        TensorInfo yi = make_info(p->y, full, 0, 0, false);
        ScatterNdQueueDescriptor d;
        d.m_Parameters = ScatterNdDescriptor(static_cast<ScatterNdFunction>(p->function), p->x.data != nullptr);
        std::vector<int32_t> shapeValues(dims, dims + p->nd + 1);
        if (p->x.data) { h.in(d, make_info(p->x, full, 0, 0, false), p->x.data); }
        else { h.in(d, TensorInfo(TensorShape({(unsigned)p->nd + 1}), DataType::Signed32), shapeValues.data()); }
        h.in(d, ii, p->indices);
        h.in(d, ui, p->updates.data);
        auto* o = h.out(d, yi);
        h.run(LayerType::ScatterNd, d);
        copy_out(o, const_cast<void*>(p->y.data), yi.GetNumBytes());
    });
}
