// Workloads of the B200Acc backend: one per layer type on the quantised hot path, each one call of the libb200k
// C ABI (include/b200k.h) on the backend's CUDA stream, plus the workload factory that creates them.
//
// A workload fills its parameter struct once, in its constructor, from the queue descriptor and the WorkloadInfo
// (exactly the information the CpuRef workload of the same layer reads in Execute), resolves device pointers from
// the tensor handles at Execute time, and launches asynchronously.  Nothing here computes on the CPU.
#include "B200Workloads.hpp"

#include <armnn/Exceptions.hpp>
#include <armnn/backends/MemCopyWorkload.hpp>
#include <armnn/backends/TensorHandle.hpp>
#include <armnn/utility/PolymorphicDowncast.hpp>
#include <backendsCommon/MemImportWorkload.hpp>
#include <backendsCommon/MemSyncWorkload.hpp>

#include <Profiling.hpp>

#include <cstring>
#include <functional>
#include <mutex>

#include "B200Timer.hpp"
#include "b200k.h"

namespace armnn
{

namespace
{

int ToB200k(DataType t)
{
    switch (t)
    {
        case DataType::Boolean:                           // one byte per element; Operand() gives it scale 1, zero point 0
        case DataType::QAsymmU8: return B200K_U8;
        case DataType::QAsymmS8:
        case DataType::QSymmS8:  return B200K_S8;
        case DataType::QSymmS16: return B200K_S16;
        case DataType::Signed32: return B200K_S32;
        case DataType::Float32:  return B200K_F32;
        default: throw InvalidArgumentException("B200Acc: unsupported data type");
    }
}

void* Dev(const ITensorHandle* h)
{
    return PolymorphicDowncast<const B200TensorHandle*>(h)->Device();
}

void Written(const ITensorHandle* h)
{
    PolymorphicDowncast<const B200TensorHandle*>(h)->MarkDeviceWritten();
}

using ContextPtr = std::shared_ptr<B200Context>;

// Small device arrays owned by a workload (per-axis scales, QLstm weights, packed tables, scratch), on the network's GPU.
struct DeviceBlobs
{
    explicit DeviceBlobs(ContextPtr c) : ctx(std::move(c)) {}
    ContextPtr ctx;
    std::vector<void*> ptrs;
    ~DeviceBlobs()
    {
        if (!ptrs.empty()) { cudaSetDevice(ctx->Device()); }
        for (void* p : ptrs) { cudaFree(p); }
    }
    void* Alloc(size_t bytes)
    {
        void* p = nullptr;
        ctx->MakeCurrent();
        B200Check(cudaMalloc(&p, bytes ? bytes : 16), "cudaMalloc");
        ptrs.push_back(p);
        return p;
    }
    void* Upload(const void* host, size_t bytes)
    {
        void* p = Alloc(bytes);
        B200Check(cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice), "cudaMemcpy H2D");
        return p;
    }
};

b200k_qtensor Operand(const TensorInfo& info, DeviceBlobs& blobs)
{
    b200k_qtensor t;
    std::memset(&t, 0, sizeof(t));
    t.dtype = ToB200k(info.GetDataType());
    if (info.HasMultipleQuantizationScales())
    {
        const std::vector<float> s = info.GetQuantizationScales();
        t.scales = static_cast<const float*>(blobs.Upload(s.data(), s.size() * sizeof(float)));
        t.scale = 1.0f;
        t.zero_point = 0;
    }
    else if (IsQuantizedType(info.GetDataType()) || info.GetDataType() == DataType::Signed32)
    {
        t.scale = info.GetQuantizationScale();
        t.zero_point = info.GetQuantizationOffset();
    }
    else
    {
        t.scale = 1.0f;
    }
    return t;
}

void Clamp(const ActivationDescriptor* act, const TensorInfo& out, int32_t& lo, int32_t& hi)
{
    int kind = 0;
    float a = 0.f, b = 0.f;
    if (act)
    {
        if (act->m_Function == ActivationFunction::ReLu) { kind = 1; }
        else if (act->m_Function == ActivationFunction::BoundedReLu) { kind = 2; a = act->m_A; b = act->m_B; }
        else { throw InvalidArgumentException("B200Acc: only ReLu / BoundedReLu can be fused"); }
    }
    B200CheckStatus(b200k_activation_clamp(kind, a, b, out.GetQuantizationScale(), out.GetQuantizationOffset(),
                                           ToB200k(out.GetDataType()), &lo, &hi));
}

// Generic workload: `launch` is built by the factory and owns everything it needs.  Execute() hands the launch to the
// network's context, which runs it on the network's stream, records it into the CUDA graph of the workload queue, or
// skips it because the graph launched by the queue's first workload already contains it.  With the Arm NN profiler
// enabled the launch is bracketed by a profiling event that carries the host wall clock and the device time.
template <typename QueueDescriptor>
class B200Workload : public BaseWorkload<QueueDescriptor>
{
public:
    using Launch = std::function<void(const QueueDescriptor&, cudaStream_t)>;
    B200Workload(const QueueDescriptor& d, const WorkloadInfo& info, ContextPtr ctx, Launch launch, bool launchesEveryInference = true)
        : BaseWorkload<QueueDescriptor>(d, info), m_Ctx(std::move(ctx)), m_Launch(std::move(launch))
    {
        m_Index = m_Ctx->Register(launchesEveryInference);
    }
    void Execute() const override
    {
        ARMNN_SCOPED_PROFILING_EVENT_WITH_INSTRUMENTS(BackendId(B200BackendId()), this->GetGuid(), this->GetName() + "_Execute",
                                                      WallClockTimer(), CudaEventTimer(m_Ctx->Stream(), m_Ctx->Device()));
        std::vector<const B200TensorHandle*> reads;
        reads.reserve(this->m_Data.m_Inputs.size());
        for (ITensorHandle* h : this->m_Data.m_Inputs) { reads.push_back(PolymorphicDowncast<const B200TensorHandle*>(h)); }
        m_Ctx->Run(m_Index, reads, [this](cudaStream_t s) { m_Launch(this->m_Data, s); });
        for (ITensorHandle* h : this->m_Data.m_Outputs) { Written(h); }
    }
    // handles are resolved at Execute time, so the core may swap in its pre-imported handles
    // (src/armnn/LoadedNetwork.cpp:821-833, 877-894); a recorded graph holds the old addresses and is dropped
    bool SupportsTensorHandleReplacement() const override { return true; }
    void ReplaceInputTensorHandle(ITensorHandle* h, unsigned int slot) override { this->m_Data.m_Inputs[slot] = h; m_Ctx->Invalidate(); }
    void ReplaceOutputTensorHandle(ITensorHandle* h, unsigned int slot) override { this->m_Data.m_Outputs[slot] = h; m_Ctx->Invalidate(); }
private:
    ContextPtr m_Ctx;
    Launch m_Launch;
    int m_Index = 0;
};

template <typename QD>
std::unique_ptr<IWorkload> Make(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx,
                                typename B200Workload<QD>::Launch fn, bool launchesEveryInference = true)
{
    return std::make_unique<B200Workload<QD>>(*PolymorphicDowncast<const QD*>(&d), info, ctx, std::move(fn), launchesEveryInference);
}

// ---- Concat, Splitter, Permute, Transpose, StridedSlice, Slice: rectangular view copies (b200k_view_copy_q) ----------
// The descriptor arithmetic is the reference's (Concatenate.cpp:14-85, Splitter.cpp:18-93, src/armnnUtils/Permute.cpp,
// Transpose.cpp, src/armnn/Descriptors.cpp:393-453 with workloads/StridedSlice.cpp:188-222, workloads/Slice.cpp:14-147);
// armnn_b200/views.py states the same rules for the Python mirror.
struct ViewOp
{
    b200k_view_copy_params p;
    unsigned int src, dst;          // index of the workload's input / output tensor
    const void* fixedSrc;           // non-null: a device constant owned by the workload instead of input `src`
};

struct ViewState
{
    explicit ViewState(const ContextPtr& ctx) : blobs(ctx) {}
    std::vector<ViewOp> ops;
    DeviceBlobs blobs;
};

void DenseStrides(const TensorShape& shape, int64_t* strides)
{
    int64_t st = 1;
    for (unsigned int d = shape.GetNumDimensions(); d-- > 0;) { strides[d] = st; st *= shape[d]; }
}

/// outer x axis x inner: the tensor seen as independent rows along `axis` (negative: counted from the end).
void RowsOf(const TensorShape& shape, int axis, int32_t& outer, int32_t& axisSize, int32_t& inner)
{
    const int rank = static_cast<int>(shape.GetNumDimensions());
    if (axis < 0) { axis += rank; }
    if (axis < 0 || axis >= rank) { throw InvalidArgumentException("B200Acc: axis outside the tensor's dimensions"); }
    outer = 1; inner = 1;
    for (int i = 0; i < axis; ++i) { outer *= static_cast<int32_t>(shape[static_cast<unsigned int>(i)]); }
    for (int i = axis + 1; i < rank; ++i) { inner *= static_cast<int32_t>(shape[static_cast<unsigned int>(i)]); }
    axisSize = static_cast<int32_t>(shape[static_cast<unsigned int>(axis)]);
}

ViewOp NewViewOp(const TensorInfo& x, const TensorInfo& y, DeviceBlobs& blobs, unsigned int src, unsigned int dst, unsigned int rank)
{
    if (rank < 1 || rank > 6) { throw InvalidArgumentException("B200Acc: view copies need a rank between 1 and 6"); }
    ViewOp op;
    std::memset(&op, 0, sizeof(op));
    op.p.x = Operand(x, blobs); op.p.y = Operand(y, blobs);
    op.p.rank = static_cast<int32_t>(rank);
    op.src = src; op.dst = dst;
    return op;
}

template <typename QD>
std::unique_ptr<IWorkload> MakeViews(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx, std::shared_ptr<ViewState> st)
{
    return Make<QD>(d, info, ctx, [st](const QD& data, cudaStream_t s)
    {
        for (ViewOp& op : st->ops)
        {
            op.p.x.data = op.fixedSrc ? op.fixedSrc : Dev(data.m_Inputs[op.src]);
            op.p.y.data = Dev(data.m_Outputs[op.dst]);
            B200CheckStatus(b200k_view_copy_q(&op.p, s));
        }
    });
}

// Concat: input v (dense) -> the block of the output at its view origin.  Where views overlap the reference lets the
// first one win, so the copies are issued last view first.
std::unique_ptr<IWorkload> MakeConcat(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx)
{
    const auto& qd = *PolymorphicDowncast<const ConcatQueueDescriptor*>(&d);
    auto st = std::make_shared<ViewState>(ctx);
    const TensorInfo& out = info.m_OutputTensorInfos[0];
    const unsigned int rank = out.GetNumDimensions();
    int64_t os[6];
    DenseStrides(out.GetShape(), os);
    for (size_t v = qd.m_ViewOrigins.size(); v-- > 0;)
    {
        const TensorInfo& in = info.m_InputTensorInfos[v];
        if (in.GetNumDimensions() != rank || qd.m_ViewOrigins[v].m_Origin.size() != rank) { throw InvalidArgumentException("B200Acc: Concat views must have the output's rank"); }
        ViewOp op = NewViewOp(in, out, st->blobs, static_cast<unsigned int>(v), 0, rank);
        DenseStrides(in.GetShape(), op.p.src_strides);
        for (unsigned int i = 0; i < rank; ++i)
        {
            const unsigned int o = qd.m_ViewOrigins[v].m_Origin[i];
            if (o + in.GetShape()[i] > out.GetShape()[i]) { throw InvalidArgumentException("B200Acc: Concat view outside the output"); }
            op.p.shape[i] = static_cast<int32_t>(in.GetShape()[i]);
            op.p.dst_strides[i] = os[i];
            op.p.dst_offset += static_cast<int64_t>(o) * os[i];
        }
        st->ops.push_back(op);
    }
    return MakeViews<ConcatQueueDescriptor>(d, info, ctx, st);
}

// Splitter: the block of the input at view v's origin -> output v (dense).
std::unique_ptr<IWorkload> MakeSplitter(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx)
{
    const auto& qd = *PolymorphicDowncast<const SplitterQueueDescriptor*>(&d);
    auto st = std::make_shared<ViewState>(ctx);
    const TensorInfo& in = info.m_InputTensorInfos[0];
    const unsigned int rank = in.GetNumDimensions();
    int64_t is[6];
    DenseStrides(in.GetShape(), is);
    for (size_t v = 0; v < qd.m_ViewOrigins.size(); ++v)
    {
        const TensorInfo& out = info.m_OutputTensorInfos[v];
        if (out.GetNumDimensions() != rank || qd.m_ViewOrigins[v].m_Origin.size() != rank) { throw InvalidArgumentException("B200Acc: Splitter views must have the input's rank"); }
        ViewOp op = NewViewOp(in, out, st->blobs, 0, static_cast<unsigned int>(v), rank);
        DenseStrides(out.GetShape(), op.p.dst_strides);
        for (unsigned int i = 0; i < rank; ++i)
        {
            const unsigned int o = qd.m_ViewOrigins[v].m_Origin[i];
            if (o + out.GetShape()[i] > in.GetShape()[i]) { throw InvalidArgumentException("B200Acc: Splitter view outside the input"); }
            op.p.shape[i] = static_cast<int32_t>(out.GetShape()[i]);
            op.p.src_strides[i] = is[i];
            op.p.src_offset += static_cast<int64_t>(o) * is[i];
        }
        st->ops.push_back(op);
    }
    return MakeViews<SplitterQueueDescriptor>(d, info, ctx, st);
}

// Permute (mappings[i]: destination dimension of source dimension i) and Transpose (mappings[i]: source dimension of
// destination dimension i): the source strides in the destination's order of dimensions.
template <typename QD>
std::unique_ptr<IWorkload> MakePermute(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx, bool transpose)
{
    const auto& qd = *PolymorphicDowncast<const QD*>(&d);
    const PermutationVector& m = qd.m_Parameters.m_DimMappings;
    auto st = std::make_shared<ViewState>(ctx);
    const TensorInfo& in = info.m_InputTensorInfos[0];
    const TensorInfo& out = info.m_OutputTensorInfos[0];
    const unsigned int rank = in.GetNumDimensions();
    if (m.GetSize() != rank || out.GetNumDimensions() != rank) { throw InvalidArgumentException("B200Acc: permutation and tensor ranks differ"); }
    int64_t is[6];
    DenseStrides(in.GetShape(), is);
    ViewOp op = NewViewOp(in, out, st->blobs, 0, 0, rank);
    DenseStrides(out.GetShape(), op.p.dst_strides);
    unsigned int srcOfDst[6] = {0, 0, 0, 0, 0, 0};
    for (unsigned int i = 0; i < rank; ++i)
    {
        if (transpose) { srcOfDst[i] = m[i]; } else { srcOfDst[m[i]] = i; }
    }
    for (unsigned int j = 0; j < rank; ++j)
    {
        if (out.GetShape()[j] != in.GetShape()[srcOfDst[j]]) { throw InvalidArgumentException("B200Acc: output shape is not the permuted input shape"); }
        op.p.shape[j] = static_cast<int32_t>(out.GetShape()[j]);
        op.p.src_strides[j] = is[srcOfDst[j]];
    }
    st->ops.push_back(op);
    return MakeViews<QD>(d, info, ctx, st);
}

// StridedSlice with begin / end / shrink-axis masks (layer support refuses ellipsis and new-axis masks).
std::unique_ptr<IWorkload> MakeStridedSlice(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx)
{
    const auto& qd = *PolymorphicDowncast<const StridedSliceQueueDescriptor*>(&d);
    const StridedSliceDescriptor& prm = qd.m_Parameters;
    auto st = std::make_shared<ViewState>(ctx);
    const TensorInfo& in = info.m_InputTensorInfos[0];
    const TensorInfo& out = info.m_OutputTensorInfos[0];
    const unsigned int rank = in.GetNumDimensions();
    if (prm.m_Begin.size() != rank || prm.m_End.size() != rank || prm.m_Stride.size() != rank) { throw InvalidArgumentException("B200Acc: StridedSlice needs begin / end / stride per input dimension"); }
    int64_t is[6];
    DenseStrides(in.GetShape(), is);
    ViewOp op = NewViewOp(in, out, st->blobs, 0, 0, rank);
    int64_t count = 1;
    for (unsigned int i = 0; i < rank; ++i)
    {
        const int stride = prm.m_Stride[i];
        if (stride == 0) { throw InvalidArgumentException("B200Acc: StridedSlice stride 0"); }
        const int start = prm.GetStartForAxis(in.GetShape(), i);
        const int stop = prm.GetStopForAxis(in.GetShape(), i, start);
        int n = 0;
        if (stride > 0 && stop > start) { n = (stop - start + stride - 1) / stride; }
        if (stride < 0 && stop < start) { n = (start - stop - stride - 1) / (-stride); }
        op.p.shape[i] = n;
        op.p.src_strides[i] = is[i] * stride;
        op.p.src_offset += static_cast<int64_t>(start) * is[i];
        count *= n;
    }
    if (static_cast<unsigned int>(count) != out.GetNumElements()) { throw InvalidArgumentException("B200Acc: StridedSlice output shape does not match the slice"); }
    int64_t st1 = 1;
    for (unsigned int i = rank; i-- > 0;) { op.p.dst_strides[i] = st1; st1 *= op.p.shape[i]; }
    st->ops.push_back(op);
    return MakeViews<StridedSliceQueueDescriptor>(d, info, ctx, st);
}

// One view over a walk of up to six dimensions given as (extent, source stride) pairs; the destination is dense.
template <typename QD>
std::unique_ptr<IWorkload> MakeWalk(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx,
                                    const std::vector<std::pair<int64_t, int64_t>>& walk)
{
    auto st = std::make_shared<ViewState>(ctx);
    ViewOp op = NewViewOp(info.m_InputTensorInfos[0], info.m_OutputTensorInfos[0], st->blobs, 0, 0, static_cast<unsigned int>(walk.size()));
    int64_t count = 1, dstStride = 1;
    for (size_t i = walk.size(); i-- > 0;)
    {
        op.p.shape[i] = static_cast<int32_t>(walk[i].first);
        op.p.src_strides[i] = walk[i].second;
        op.p.dst_strides[i] = dstStride;
        dstStride *= walk[i].first;
        count *= walk[i].first;
    }
    if (static_cast<unsigned int>(count) != info.m_OutputTensorInfos[0].GetNumElements() ||
        info.m_InputTensorInfos[0].GetNumElements() != info.m_OutputTensorInfos[0].GetNumElements())
    {
        throw InvalidArgumentException("B200Acc: output shape does not match the layer's rearrangement of the input");
    }
    st->ops.push_back(op);
    return MakeViews<QD>(d, info, ctx, st);
}

// DepthToSpace (workloads/DepthToSpace.cpp:15-100) and SpaceToDepth (workloads/SpaceToDepth.cpp:42-104), both layouts.
template <typename QD>
std::unique_ptr<IWorkload> MakeDepthSpace(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx, bool toSpace)
{
    const auto& qd = *PolymorphicDowncast<const QD*>(&d);
    const TensorShape& s = info.m_InputTensorInfos[0].GetShape();
    if (s.GetNumDimensions() != 4 || qd.m_Parameters.m_BlockSize == 0) { throw InvalidArgumentException("B200Acc: DepthToSpace / SpaceToDepth need 4-D tensors and a block size"); }
    const bool nchw = qd.m_Parameters.m_DataLayout == DataLayout::NCHW;
    const int64_t b = qd.m_Parameters.m_BlockSize;
    int64_t is[6];
    DenseStrides(s, is);
    const int64_t n = s[0], c = nchw ? s[1] : s[3], h = nchw ? s[2] : s[1], w = nchw ? s[3] : s[2];
    if (toSpace)
    {
        if (c % (b * b) != 0) { throw InvalidArgumentException("B200Acc: DepthToSpace channels are not a multiple of the block size squared"); }
        const int64_t co = c / (b * b);
        if (nchw) { return MakeWalk<QD>(d, info, ctx, {{n, is[0]}, {co, is[1]}, {h, is[2]}, {b, b * co * is[1]}, {w, is[3]}, {b, co * is[1]}}); }
        return MakeWalk<QD>(d, info, ctx, {{n, is[0]}, {h, is[1]}, {b, b * co}, {w, is[2]}, {b, co}, {co, 1}});
    }
    if (h % b != 0 || w % b != 0) { throw InvalidArgumentException("B200Acc: SpaceToDepth height / width are not multiples of the block size"); }
    if (nchw) { return MakeWalk<QD>(d, info, ctx, {{n, is[0]}, {b, is[2]}, {b, is[3]}, {c, is[1]}, {h / b, b * is[2]}, {w / b, b * is[3]}}); }
    return MakeWalk<QD>(d, info, ctx, {{n, is[0]}, {h / b, b * is[1]}, {w / b, b * is[2]}, {b, is[1]}, {b, is[2]}, {c, 1}});
}

// BatchToSpaceNd (workloads/BatchToSpaceNd.cpp:50-117) and SpaceToBatchNd (workloads/SpaceToBatchNd.cpp:49-131), ranks 3
// and 4, both layouts.  With the batch-side tensor B [nb * bh * bw, hb, wb, c] and the space-side tensor S [nb, hs, ws, c],
// batch (i * bw + j) * nb + b of B pairs its pixel (y, x) with pixel (y * bh + i - top, x * bw + j - left) of S: one
// strided block per (i, j).  BatchToSpaceNd copies B -> S (top / left: crops); SpaceToBatchNd copies S -> B (top / left:
// padding) after filling B with its encoding of 0.0 when there is any padding.
template <typename QD>
std::unique_ptr<IWorkload> MakeBatchSpace(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx,
                                          const std::vector<unsigned int>& block,
                                          const std::vector<std::pair<unsigned int, unsigned int>>& edges, DataLayout layout, bool toSpace)
{
    auto st = std::make_shared<ViewState>(ctx);
    const TensorInfo& in = info.m_InputTensorInfos[0];
    const TensorInfo& out = info.m_OutputTensorInfos[0];
    const TensorInfo& B = toSpace ? in : out;
    const TensorInfo& S = toSpace ? out : in;
    const unsigned int rank = in.GetNumDimensions();
    if ((rank != 3 && rank != 4) || out.GetNumDimensions() != rank || block.size() != rank - 2 || edges.size() != rank - 2)
    {
        throw InvalidArgumentException("B200Acc: BatchToSpaceNd / SpaceToBatchNd need 3 or 4 dimensions and one block extent per spatial dimension");
    }
    const bool nchw = layout == DataLayout::NCHW;
    const unsigned int hI = nchw ? 2 : 1, wI = nchw ? 3 : 2, cI = nchw ? 1 : rank - 1;
    auto dim = [&](const TensorInfo& t, unsigned int i) { return (i < rank) ? static_cast<int64_t>(t.GetShape()[i]) : int64_t(1); };
    int64_t bs[6] = {0, 0, 0, 0, 0, 0}, ss[6] = {0, 0, 0, 0, 0, 0};
    DenseStrides(B.GetShape(), bs);
    DenseStrides(S.GetShape(), ss);
    const bool hasW = rank == 4;
    const int64_t bh = block[0], bw = hasW ? block[1] : 1;
    const int64_t top = edges[0].first, bottom = edges[0].second, left = hasW ? edges[1].first : 0, right = hasW ? edges[1].second : 0;
    const int64_t nb = dim(S, 0), hb = dim(B, hI), wb = hasW ? dim(B, wI) : 1, c = dim(B, cI);
    const int64_t hs = dim(S, hI), wsz = hasW ? dim(S, wI) : 1;
    if (bh < 1 || bw < 1 || dim(B, 0) != nb * bh * bw || dim(S, cI) != c || hb * bh != hs + top + bottom || wb * bw != wsz + left + right)
    {
        throw InvalidArgumentException("B200Acc: BatchToSpaceNd / SpaceToBatchNd shapes do not match the block shape and crops / padding");
    }
    const int64_t bsH = bs[hI], bsW = hasW ? bs[wI] : 0, bsC = bs[cI], ssH = ss[hI], ssW = hasW ? ss[wI] : 0, ssC = ss[cI];
    if (!toSpace && (top || bottom || left || right))
    {
        // every element of the output <- one element holding Q_out(0.0) (source strides 0)
        uint8_t zero[4] = {0, 0, 0, 0};
        const DataType t = out.GetDataType();
        if (t == DataType::QSymmS16)
        {
            const int16_t v = static_cast<int16_t>(std::min(std::max(out.GetQuantizationOffset(), -32768), 32767));
            std::memcpy(zero, &v, 2);
        }
        else if (t == DataType::QAsymmU8) { zero[0] = static_cast<uint8_t>(std::min(std::max(out.GetQuantizationOffset(), 0), 255)); }
        else if (t == DataType::QAsymmS8 || t == DataType::QSymmS8)
        {
            zero[0] = static_cast<uint8_t>(static_cast<int8_t>(std::min(std::max(out.GetQuantizationOffset(), -128), 127)));
        }
        ViewOp op = NewViewOp(out, out, st->blobs, 0, 0, rank);
        op.fixedSrc = st->blobs.Upload(zero, sizeof(zero));
        DenseStrides(out.GetShape(), op.p.dst_strides);
        for (unsigned int i = 0; i < rank; ++i) { op.p.shape[i] = static_cast<int32_t>(out.GetShape()[i]); }
        st->ops.push_back(op);
    }
    auto span = [](int64_t loNum, int64_t hiNum, int64_t blk, int64_t limit, int64_t& first, int64_t& count)
    {
        // indices n in [0, limit) with loNum <= n * blk <= hiNum
        first = loNum <= 0 ? 0 : (loNum + blk - 1) / blk;
        const int64_t last = hiNum < 0 ? -1 : std::min(limit - 1, hiNum / blk);
        count = std::max<int64_t>(0, last - first + 1);
    };
    for (int64_t i = 0; i < bh; ++i)
    {
        int64_t h0, nh;
        span(top - i, hs - 1 + top - i, bh, hb, h0, nh);
        for (int64_t j = 0; j < bw; ++j)
        {
            int64_t w0, nw;
            span(left - j, wsz - 1 + left - j, bw, wb, w0, nw);
            if (nh == 0 || nw == 0) { continue; }
            // the walk in the destination's memory order: (batch, h, w, c) for NHWC, (batch, c, h, w) for NCHW
            const int64_t ext[4] = {nb, nh, nw, c};
            const int64_t bStr[4] = {bs[0], bsH, bsW, bsC}, sStr[4] = {ss[0], ssH * bh, ssW * bw, ssC};
            const int64_t bOff = (i * bw + j) * nb * bs[0] + h0 * bsH + w0 * bsW;
            const int64_t sOff = (h0 * bh + i - top) * ssH + (w0 * bw + j - left) * ssW;
            const int orderNhwc[4] = {0, 1, 2, 3}, orderNchw[4] = {0, 3, 1, 2};
            const int* order = nchw ? orderNchw : orderNhwc;
            ViewOp op = NewViewOp(in, out, st->blobs, 0, 0, 4);
            for (int k = 0; k < 4; ++k)
            {
                op.p.shape[k] = static_cast<int32_t>(ext[order[k]]);
                op.p.src_strides[k] = toSpace ? bStr[order[k]] : sStr[order[k]];
                op.p.dst_strides[k] = toSpace ? sStr[order[k]] : bStr[order[k]];
            }
            op.p.src_offset = toSpace ? bOff : sOff;
            op.p.dst_offset = toSpace ? sOff : bOff;
            st->ops.push_back(op);
        }
    }
    return MakeViews<QD>(d, info, ctx, st);
}

/// Appends one dimension to a view, dropping extents of 1 and folding a dimension into its outer neighbour when the two
/// are contiguous on both sides, so that walks over pairs of dimensions (Tile) fit the kernel's six.
void PushDim(ViewOp& op, int64_t extent, int64_t srcStride, int64_t dstStride)
{
    if (extent == 1) { return; }
    const int r = op.p.rank;
    if (r > 0 && op.p.src_strides[r - 1] == srcStride * extent && op.p.dst_strides[r - 1] == dstStride * extent)
    {
        op.p.shape[r - 1] = static_cast<int32_t>(op.p.shape[r - 1] * extent);
        op.p.src_strides[r - 1] = srcStride; op.p.dst_strides[r - 1] = dstStride;
        return;
    }
    if (r >= 6) { throw InvalidArgumentException("B200Acc: the rearrangement needs more than six dimensions"); }
    op.p.shape[r] = static_cast<int32_t>(extent); op.p.src_strides[r] = srcStride; op.p.dst_strides[r] = dstStride;
    op.p.rank = r + 1;
}

void FinishDims(ViewOp& op)
{
    if (op.p.rank == 0) { op.p.rank = 1; op.p.shape[0] = 1; op.p.src_strides[0] = 1; op.p.dst_strides[0] = 1; }
}

// Tile (workloads/Tile.cpp:47-103): every dimension becomes a (repeat, size) pair whose repeat part has source stride 0.
std::unique_ptr<IWorkload> MakeTile(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx)
{
    const auto& qd = *PolymorphicDowncast<const TileQueueDescriptor*>(&d);
    auto st = std::make_shared<ViewState>(ctx);
    const TensorInfo& in = info.m_InputTensorInfos[0];
    const TensorInfo& out = info.m_OutputTensorInfos[0];
    const unsigned int rank = in.GetNumDimensions();
    if (qd.m_Parameters.m_Multiples.size() != rank || out.GetNumDimensions() != rank || rank > 6) { throw InvalidArgumentException("B200Acc: Tile needs one multiple per dimension"); }
    int64_t is[6], os[6];
    DenseStrides(in.GetShape(), is);
    DenseStrides(out.GetShape(), os);
    ViewOp op = NewViewOp(in, out, st->blobs, 0, 0, 1);
    op.p.rank = 0;
    for (unsigned int i = 0; i < rank; ++i)
    {
        const int64_t m = qd.m_Parameters.m_Multiples[i], n = in.GetShape()[i];
        if (m < 1 || out.GetShape()[i] != n * m) { throw InvalidArgumentException("B200Acc: Tile output shape is not input shape x multiples"); }
        PushDim(op, m, 0, n * os[i]);
        PushDim(op, n, is[i], os[i]);
    }
    FinishDims(op);
    st->ops.push_back(op);
    return MakeViews<TileQueueDescriptor>(d, info, ctx, st);
}

// BroadcastTo (RefBroadcastToWorkload.cpp:29-44): the input aligned to the innermost dimensions of the output, extents of
// 1 (or absent dimensions) repeated with source stride 0.
std::unique_ptr<IWorkload> MakeBroadcastTo(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx)
{
    auto st = std::make_shared<ViewState>(ctx);
    const TensorInfo& in = info.m_InputTensorInfos[0];
    const TensorInfo& out = info.m_OutputTensorInfos[0];
    const unsigned int ir = in.GetNumDimensions(), orank = out.GetNumDimensions();
    if (ir > orank || orank > 6) { throw InvalidArgumentException("B200Acc: BroadcastTo needs an output of at least the input's rank (at most 6)"); }
    int64_t is[6], os[6];
    DenseStrides(in.GetShape(), is);
    DenseStrides(out.GetShape(), os);
    ViewOp op = NewViewOp(in, out, st->blobs, 0, 0, 1);
    op.p.rank = 0;
    for (unsigned int i = 0; i < orank; ++i)
    {
        const int id = static_cast<int>(i) - static_cast<int>(orank - ir);
        const int64_t n = id < 0 ? 1 : static_cast<int64_t>(in.GetShape()[static_cast<unsigned int>(id)]);
        if (n != 1 && n != out.GetShape()[i]) { throw InvalidArgumentException("B200Acc: BroadcastTo shapes are not compatible"); }
        PushDim(op, out.GetShape()[i], n == 1 ? 0 : is[id], os[i]);
    }
    FinishDims(op);
    st->ops.push_back(op);
    return MakeViews<BroadcastToQueueDescriptor>(d, info, ctx, st);
}

// ChannelShuffle (RefChannelShuffleWorkload.cpp:28-76): output channel i g + j is input channel i + j s.
std::unique_ptr<IWorkload> MakeChannelShuffle(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx)
{
    const auto& qd = *PolymorphicDowncast<const ChannelShuffleQueueDescriptor*>(&d);
    const TensorShape& s = info.m_InputTensorInfos[0].GetShape();
    const unsigned int axis = qd.m_Parameters.m_Axis, g = qd.m_Parameters.m_NumGroups;
    if (axis >= s.GetNumDimensions() || g == 0 || s[axis] % g != 0) { throw InvalidArgumentException("B200Acc: ChannelShuffle groups do not divide the channel count"); }
    int64_t outer = 1, inner = 1;
    for (unsigned int i = 0; i < axis; ++i) { outer *= s[i]; }
    for (unsigned int i = axis + 1; i < s.GetNumDimensions(); ++i) { inner *= s[i]; }
    const int64_t size = s[axis] / g;
    return MakeWalk<ChannelShuffleQueueDescriptor>(d, info, ctx, {{outer, s[axis] * inner}, {size, inner}, {g, size * inner}, {inner, 1}});
}

// Stack (workloads/Stack.cpp:14-120): input i becomes index i of the new dimension.
std::unique_ptr<IWorkload> MakeStack(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx)
{
    const auto& qd = *PolymorphicDowncast<const StackQueueDescriptor*>(&d);
    auto st = std::make_shared<ViewState>(ctx);
    const TensorInfo& out = info.m_OutputTensorInfos[0];
    const unsigned int axis = qd.m_Parameters.m_Axis, inRank = info.m_InputTensorInfos[0].GetNumDimensions();
    if (axis > inRank || out.GetNumDimensions() != inRank + 1 || inRank + 1 > 6) { throw InvalidArgumentException("B200Acc: Stack axis or rank not supported"); }
    int64_t os[6];
    DenseStrides(out.GetShape(), os);
    for (unsigned int v = 0; v < info.m_InputTensorInfos.size(); ++v)
    {
        const TensorInfo& in = info.m_InputTensorInfos[v];
        if (in.GetShape() != info.m_InputTensorInfos[0].GetShape()) { throw InvalidArgumentException("B200Acc: Stack inputs must share one shape"); }
        ViewOp op = NewViewOp(in, out, st->blobs, v, 0, inRank);
        DenseStrides(in.GetShape(), op.p.src_strides);
        for (unsigned int i = 0; i < inRank; ++i)
        {
            op.p.shape[i] = static_cast<int32_t>(in.GetShape()[i]);
            op.p.dst_strides[i] = os[i < axis ? i : i + 1];
        }
        op.p.dst_offset = static_cast<int64_t>(v) * os[axis];
        st->ops.push_back(op);
    }
    return MakeViews<StackQueueDescriptor>(d, info, ctx, st);
}

std::unique_ptr<IWorkload> MakeSlice(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx)
{
    const auto& qd = *PolymorphicDowncast<const SliceQueueDescriptor*>(&d);
    auto st = std::make_shared<ViewState>(ctx);
    const TensorInfo& in = info.m_InputTensorInfos[0];
    const TensorInfo& out = info.m_OutputTensorInfos[0];
    const unsigned int rank = in.GetNumDimensions();
    if (qd.m_Parameters.m_Begin.size() != rank || qd.m_Parameters.m_Size.size() != rank || out.GetNumDimensions() != rank) { throw InvalidArgumentException("B200Acc: Slice needs begin / size per input dimension"); }
    int64_t is[6];
    DenseStrides(in.GetShape(), is);
    ViewOp op = NewViewOp(in, out, st->blobs, 0, 0, rank);
    DenseStrides(out.GetShape(), op.p.dst_strides);
    for (unsigned int i = 0; i < rank; ++i)
    {
        const unsigned int b = qd.m_Parameters.m_Begin[i], n = qd.m_Parameters.m_Size[i];
        if (b + n > in.GetShape()[i] || n != out.GetShape()[i]) { throw InvalidArgumentException("B200Acc: Slice block outside the input"); }
        op.p.shape[i] = static_cast<int32_t>(n);
        op.p.src_strides[i] = is[i];
        op.p.src_offset += static_cast<int64_t>(b) * is[i];
    }
    st->ops.push_back(op);
    return MakeViews<SliceQueueDescriptor>(d, info, ctx, st);
}

struct ConvState
{
    explicit ConvState(const ContextPtr& ctx) : blobs(ctx) {}
    b200k_conv2d_params p;
    DeviceBlobs blobs;
    void* packed = nullptr;
    std::once_flag once;
};

// Geometry, quantisation and buffers of a convolution from the layer's descriptor and tensor infos
// (data, weights[, bias] -> y); `act` clamps y, or the fused Add's output when there is one.
template <typename Descriptor>
void FillConv(ConvState& st, const Descriptor& prm, const TensorInfo& x, const TensorInfo& w, const TensorInfo* bias,
              const TensorInfo& y, bool depthwise)
{
    if (prm.m_DataLayout != DataLayout::NHWC) { throw InvalidArgumentException("B200Acc: NHWC only"); }
    b200k_conv2d_params& p = st.p;
    std::memset(&p, 0, sizeof(p));
    p.x = Operand(x, st.blobs);
    p.w = Operand(w, st.blobs);
    p.y = Operand(y, st.blobs);
    if (prm.m_BiasEnabled && bias) { p.bias = Operand(*bias, st.blobs); }
    p.n = x.GetShape()[0]; p.h = x.GetShape()[1]; p.wd = x.GetShape()[2]; p.c = x.GetShape()[3];
    p.oh = y.GetShape()[1]; p.ow = y.GetShape()[2]; p.oc = y.GetShape()[3];
    p.kh = w.GetShape()[1]; p.kw = w.GetShape()[2];
    p.stride_h = prm.m_StrideY; p.stride_w = prm.m_StrideX;
    p.pad_top = prm.m_PadTop; p.pad_left = prm.m_PadLeft;
    p.dil_h = prm.m_DilationY; p.dil_w = prm.m_DilationX;
    p.selftest_us = st.blobs.ctx->SelfTestUs();
    if (!depthwise)
    {
        st.packed = st.blobs.Alloc(b200k_conv2d_pack_bytes(p.oc, p.kh, p.kw, p.c));
        const size_t scratch = b200k_conv2d_scratch_bytes(&p);
        if (scratch) { p.scratch = st.blobs.Alloc(scratch); p.scratch_bytes = scratch; }
    }
}

// The weight bytes reach the device when the Constant workloads run, which is after workload creation and
// PostAllocationConfigure (src/armnn/LoadedNetwork.cpp:559-568): build the weight table on first use.
void LaunchConv(ConvState& st, cudaStream_t s)
{
    b200k_conv2d_params& q = st.p;
    std::call_once(st.once, [&] { B200CheckStatus(b200k_conv2d_pack(&q, st.packed, s)); q.packed = st.packed; });
    B200CheckStatus(b200k_conv2d_q8(&q, s));
}

// NCHW tensors around the NHWC kernels: a layer that arrives in NCHW (the ONNX and Caffe conventions) runs as
// re-layout -> NHWC kernel -> re-layout, through scratch tensors the workload owns.  The re-layouts are view copies between
// tensors of one quantisation: the bytes move as they are.
TensorInfo NhwcOf(const TensorInfo& nchw)
{
    TensorInfo t = nchw;
    const TensorShape& s = nchw.GetShape();
    t.SetShape(TensorShape({s[0], s[2], s[3], s[1]}));
    return t;
}

/// Copy of a 4-D tensor [d0, d1, d2, d3] into the order `order` of its dimensions (destination dense).
b200k_view_copy_params Relayout(const TensorInfo& src, const unsigned int (&order)[4], DeviceBlobs& blobs)
{
    b200k_view_copy_params v;
    std::memset(&v, 0, sizeof(v));
    v.x = Operand(src, blobs); v.y = v.x;
    v.rank = 4;
    int64_t ss[6];
    DenseStrides(src.GetShape(), ss);
    int64_t dst = 1;
    for (int k = 3; k >= 0; --k)
    {
        v.shape[k] = static_cast<int32_t>(src.GetShape()[order[k]]);
        v.src_strides[k] = ss[order[k]];
        v.dst_strides[k] = dst;
        dst *= v.shape[k];
    }
    return v;
}

constexpr unsigned int kNchwToNhwc[4] = {0, 2, 3, 1};
constexpr unsigned int kNhwcToNchw[4] = {0, 3, 1, 2};

struct LayoutState
{
    b200k_view_copy_params in, out, weights;      // NCHW -> NHWC input, NHWC -> NCHW output, OIHW -> OHWI weights
    void* x = nullptr; void* y = nullptr; void* w = nullptr;
};

template <typename QD>
std::unique_ptr<IWorkload> MakeConv(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx, bool depthwise)
{
    const QD& qd = *PolymorphicDowncast<const QD*>(&d);
    auto st = std::make_shared<ConvState>(ctx);
    const bool nchw = qd.m_Parameters.m_DataLayout == DataLayout::NCHW;
    auto lay = std::make_shared<LayoutState>();
    auto prm = qd.m_Parameters;
    prm.m_DataLayout = DataLayout::NHWC;
    TensorInfo xi = info.m_InputTensorInfos[0], wi = info.m_InputTensorInfos[1], yi = info.m_OutputTensorInfos[0];
    if (nchw)
    {
        lay->in = Relayout(xi, kNchwToNhwc, st->blobs);
        lay->x = st->blobs.Alloc(xi.GetNumBytes());
        xi = NhwcOf(xi);
        const TensorInfo yNhwc = NhwcOf(yi);
        lay->out = Relayout(yNhwc, kNhwcToNchw, st->blobs);
        lay->y = st->blobs.Alloc(yi.GetNumBytes());
        yi = yNhwc;
        if (!depthwise)
        {
            // Convolution2d weights are [O, I, H, W] in an NCHW layer; the depthwise ones are [1, H, W, I * M] in both layouts
            lay->weights = Relayout(wi, kNchwToNhwc, st->blobs);
            lay->w = st->blobs.Alloc(wi.GetNumBytes());
            wi = NhwcOf(wi);
        }
    }
    FillConv(*st, prm, xi, wi, info.m_InputTensorInfos.size() > 2 ? &info.m_InputTensorInfos[2] : nullptr, yi, depthwise);
    const bool f32 = yi.GetDataType() == DataType::Float32;
    // (activations are never fused into the fp32 variant: B200Backend::OptimizeSubgraphView)
    if (!f32) { Clamp(qd.template GetAdditionalInformation<ActivationDescriptor>(), yi, st->p.clamp_lo, st->p.clamp_hi); }
    const int biasType = f32 ? B200K_F32 : B200K_S32;
    return Make<QD>(d, info, ctx, [st, lay, depthwise, f32, nchw, biasType](const QD& data, cudaStream_t s)
    {
        b200k_conv2d_params& q = st->p;
        q.x.data = Dev(data.m_Inputs[0]);
        q.w.data = Dev(data.m_Inputs[1]);
        if (q.bias.dtype == biasType && data.m_Inputs.size() > 2) { q.bias.data = Dev(data.m_Inputs[2]); }
        q.y.data = Dev(data.m_Outputs[0]);
        if (nchw)
        {
            lay->in.x.data = q.x.data; lay->in.y.data = lay->x;
            B200CheckStatus(b200k_view_copy_q(&lay->in, s));
            q.x.data = lay->x;
            if (lay->w)
            {
                lay->weights.x.data = q.w.data; lay->weights.y.data = lay->w;
                B200CheckStatus(b200k_view_copy_q(&lay->weights, s));
                q.w.data = lay->w;
            }
            lay->out.x.data = lay->y; lay->out.y.data = q.y.data;
            q.y.data = lay->y;
        }
        if (f32) { B200CheckStatus(depthwise ? b200k_dwconv2d_f32(&q, s) : b200k_conv2d_f32(&q, s)); }
        else if (depthwise) { B200CheckStatus(b200k_dwconv2d_q8(&q, s)); }
        else { LaunchConv(*st, s); }
        if (nchw) { B200CheckStatus(b200k_view_copy_q(&lay->out, s)); }
    });
}

// Convolution2d -> Add [-> Activation] folded into one PreCompiled layer by B200Backend::OptimizeSubgraphView:
// inputs (data, weights[, bias], other operand), output = the Add's (Activation's) output.
std::unique_ptr<IWorkload> MakeFusedConvAdd(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx, const B200FusedConvAdd& fused)
{
    const size_t nIn = info.m_InputTensorInfos.size();
    const bool bias = fused.m_Convolution.m_BiasEnabled;
    if (nIn != (bias ? 4u : 3u) || info.m_OutputTensorInfos.size() != 1)
    {
        throw InvalidArgumentException("B200Acc: fused convolution + Add expects (data, weights[, bias], operand) -> output");
    }
    auto st = std::make_shared<ConvState>(ctx);
    const TensorInfo& other = info.m_InputTensorInfos[nIn - 1];
    const TensorInfo& out = info.m_OutputTensorInfos[0];
    FillConv(*st, fused.m_Convolution, info.m_InputTensorInfos[0], info.m_InputTensorInfos[1],
             bias ? &info.m_InputTensorInfos[2] : nullptr, fused.m_ConvolutionOutput, false);
    st->p.add_operand = Operand(other, st->blobs);
    st->p.add_out = Operand(out, st->blobs);
    Clamp(fused.m_HasActivation ? &fused.m_Activation : nullptr, out, st->p.clamp_lo, st->p.clamp_hi);
    return Make<PreCompiledQueueDescriptor>(d, info, ctx, [st, bias, nIn](const PreCompiledQueueDescriptor& data, cudaStream_t s)
    {
        b200k_conv2d_params& q = st->p;
        q.x.data = Dev(data.m_Inputs[0]);
        q.w.data = Dev(data.m_Inputs[1]);
        if (bias) { q.bias.data = Dev(data.m_Inputs[2]); }
        q.add_operand.data = Dev(data.m_Inputs[nIn - 1]);
        q.add_out.data = Dev(data.m_Outputs[0]);
        LaunchConv(*st, s);
    });
}

struct FcState
{
    explicit FcState(const ContextPtr& ctx) : blobs(ctx) {}
    b200k_fc_params p;
    DeviceBlobs blobs;
    void* packed = nullptr;
    std::once_flag once;
};

std::unique_ptr<IWorkload> MakeFc(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx)
{
    const auto& qd = *PolymorphicDowncast<const FullyConnectedQueueDescriptor*>(&d);
    auto st = std::make_shared<FcState>(ctx);
    b200k_fc_params& p = st->p;
    std::memset(&p, 0, sizeof(p));
    const TensorInfo& x = info.m_InputTensorInfos[0];
    const TensorInfo& w = info.m_InputTensorInfos[1];
    const TensorInfo& y = info.m_OutputTensorInfos[0];
    p.x = Operand(x, st->blobs);
    p.w = Operand(w, st->blobs);
    p.y = Operand(y, st->blobs);
    if (qd.m_Parameters.m_BiasEnabled) { p.bias = Operand(info.m_InputTensorInfos[2], st->blobs); }
    p.m = x.GetShape()[0];
    p.k = x.GetNumElements() / x.GetShape()[0];          // inputs of rank > 2 are flattened (FullyConnected.cpp:16-24)
    p.n = y.GetShape()[y.GetNumDimensions() - 1];
    p.transpose_w = qd.m_Parameters.m_TransposeWeightMatrix ? 1 : 0;
    if (x.GetDataType() == DataType::Float32)
    {
        // the fp32 variant (activations are never fused into it: B200Backend::OptimizeSubgraphView)
        return Make<FullyConnectedQueueDescriptor>(d, info, ctx, [st](const FullyConnectedQueueDescriptor& data, cudaStream_t s)
        {
            b200k_fc_params& q = st->p;
            q.x.data = Dev(data.m_Inputs[0]);
            q.w.data = Dev(data.m_Inputs[1]);
            if (q.bias.dtype == B200K_F32 && data.m_Inputs.size() > 2) { q.bias.data = Dev(data.m_Inputs[2]); }
            q.y.data = Dev(data.m_Outputs[0]);
            B200CheckStatus(b200k_fully_connected_f32(&q, s));
        });
    }
    Clamp(qd.GetAdditionalInformation<ActivationDescriptor>(), y, p.clamp_lo, p.clamp_hi);
    if (p.transpose_w) { st->packed = st->blobs.Alloc(b200k_conv2d_pack_bytes(p.n, 1, 1, p.k)); }
    return Make<FullyConnectedQueueDescriptor>(d, info, ctx, [st](const FullyConnectedQueueDescriptor& data, cudaStream_t s)
    {
        b200k_fc_params& q = st->p;
        q.x.data = Dev(data.m_Inputs[0]);
        q.w.data = Dev(data.m_Inputs[1]);
        if (q.bias.dtype == B200K_S32 && data.m_Inputs.size() > 2) { q.bias.data = Dev(data.m_Inputs[2]); }
        q.y.data = Dev(data.m_Outputs[0]);
        if (st->packed)
        {
            std::call_once(st->once, [&]
            {
                b200k_conv2d_params c;
                std::memset(&c, 0, sizeof(c));
                c.w = q.w; c.oc = q.n; c.kh = 1; c.kw = 1; c.c = q.k;
                B200CheckStatus(b200k_conv2d_pack(&c, st->packed, s));
                q.packed = st->packed;
            });
        }
        B200CheckStatus(b200k_fully_connected_q8(&q, s));
    });
}

template <typename P>
struct SimpleState
{
    explicit SimpleState(const ContextPtr& ctx) : blobs(ctx) {}
    P p;
    DeviceBlobs blobs;
};

// Reduce (and Mean over axes other than H and W): b200k_reduce_q over the descriptor's axes (none: all of them).
template <typename QD>
std::unique_ptr<IWorkload> MakeReduce(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx,
                                      const std::vector<unsigned int>& axes, int32_t op)
{
    auto st = std::make_shared<SimpleState<b200k_reduce_params>>(ctx);
    b200k_reduce_params& p = st->p;
    std::memset(&p, 0, sizeof(p));
    const TensorInfo& x = info.m_InputTensorInfos[0];
    p.x = Operand(x, st->blobs); p.y = Operand(info.m_OutputTensorInfos[0], st->blobs);
    p.rank = static_cast<int32_t>(x.GetNumDimensions());
    if (p.rank < 1 || p.rank > 6) { throw InvalidArgumentException("B200Acc: Reduce needs a rank between 1 and 6"); }
    for (int i = 0; i < p.rank; ++i) { p.shape[i] = static_cast<int32_t>(x.GetShape()[static_cast<unsigned int>(i)]); }
    for (unsigned int a : axes)
    {
        if (a >= x.GetNumDimensions()) { throw InvalidArgumentException("B200Acc: Reduce axis outside the tensor's rank"); }
        p.axis_mask |= 1 << a;
    }
    p.op = op;
    return Make<QD>(d, info, ctx, [st](const QD& data, cudaStream_t s)
    {
        st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
        B200CheckStatus(b200k_reduce_q(&st->p, s));
    });
}


/// The workload class is a template over the queue descriptor; the legacy layer types (Addition, Subtraction, ...) and
/// Prelu each have their own descriptor type around the same two inputs and one output.
template <typename... Ds>
struct EltwiseWrap;
template <>
struct EltwiseWrap<>
{
    template <typename Fn>
    static std::unique_ptr<IWorkload> Make(const QueueDescriptor&, const WorkloadInfo&, const ContextPtr&, Fn&&) { return nullptr; }
};
template <typename D, typename... Ds>
struct EltwiseWrap<D, Ds...>
{
    template <typename Fn>
    static std::unique_ptr<IWorkload> Make(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx, Fn&& fn)
    {
        if (auto* e = dynamic_cast<const D*>(&d)) { return std::make_unique<B200Workload<D>>(*e, info, ctx, fn); }
        return EltwiseWrap<Ds...>::Make(d, info, ctx, fn);
    }
};

/// op: armnn::BinaryOperation, or B200K_ELTWISE_PRELU with the alpha tensor as second operand.  A second operand of lower
/// rank (Prelu's alpha, src/armnn/layers/PreluLayer.cpp:38-103) is aligned to the innermost dimensions.
std::unique_ptr<IWorkload> MakeEltwise(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx, int32_t op,
                                       const ActivationDescriptor* act)
{
    auto st = std::make_shared<SimpleState<b200k_eltwise_params>>(ctx);
    b200k_eltwise_params& p = st->p;
    std::memset(&p, 0, sizeof(p));
    const TensorInfo& a = info.m_InputTensorInfos[0];
    const TensorInfo& b = info.m_InputTensorInfos[1];
    const TensorInfo& o = info.m_OutputTensorInfos[0];
    p.a = Operand(a, st->blobs); p.b = Operand(b, st->blobs); p.out = Operand(o, st->blobs);
    p.rank = static_cast<int32_t>(o.GetNumDimensions());
    const int ra = static_cast<int>(a.GetNumDimensions()), rb = static_cast<int>(b.GetNumDimensions());
    if (p.rank > 4 || ra > p.rank || rb > p.rank || ((ra != p.rank || rb != p.rank) && op != B200K_ELTWISE_PRELU))
    {
        throw InvalidArgumentException("B200Acc: elementwise operands must share a rank <= 4");
    }
    for (int i = 0; i < p.rank; ++i)
    {
        const int ia = i - (p.rank - ra), ib = i - (p.rank - rb);
        p.shape_a[i] = ia < 0 ? 1 : static_cast<int32_t>(a.GetShape()[static_cast<unsigned>(ia)]);
        p.shape_b[i] = ib < 0 ? 1 : static_cast<int32_t>(b.GetShape()[static_cast<unsigned>(ib)]);
        p.shape_out[i] = static_cast<int32_t>(o.GetShape()[static_cast<unsigned>(i)]);
    }
    p.op = op;
    if (o.GetDataType() == DataType::Boolean) { p.clamp_lo = 0; p.clamp_hi = 255; }
    else if (o.GetDataType() != DataType::Float32) { Clamp(act, o, p.clamp_lo, p.clamp_hi); }
    auto fn = [st](const QueueDescriptor& data, cudaStream_t s)
    {
        b200k_eltwise_params& q = st->p;
        q.a.data = Dev(data.m_Inputs[0]); q.b.data = Dev(data.m_Inputs[1]); q.out.data = Dev(data.m_Outputs[0]);
        B200CheckStatus(b200k_eltwise_q8(&q, s));
    };
    ARMNN_NO_DEPRECATE_WARN_BEGIN
    return EltwiseWrap<ElementwiseBinaryQueueDescriptor, AdditionQueueDescriptor, MultiplicationQueueDescriptor,
                       SubtractionQueueDescriptor, DivisionQueueDescriptor, MaximumQueueDescriptor, MinimumQueueDescriptor,
                       PreluQueueDescriptor, ComparisonQueueDescriptor, LogicalBinaryQueueDescriptor>::Make(d, info, ctx, fn);
    ARMNN_NO_DEPRECATE_WARN_END
}

// Lstm and UnidirectionalSequenceLstm on Float32 tensors: one b200k_lstm_step_f32 per time step.  LstmQueueDescriptor and
// UnidirectionalSequenceLstmQueueDescriptor carry the same members under the same names.
template <typename QD>
std::unique_ptr<IWorkload> MakeLstm(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx, bool sequence)
{
    const auto& qd = *PolymorphicDowncast<const QD*>(&d);
    const auto& prm = qd.m_Parameters;
    struct State
    {
        explicit State(const ContextPtr& c) : blobs(c) {}
        b200k_lstm_params p;
        DeviceBlobs blobs;
        int64_t steps = 1, stepIn = 0, stepOut = 0;          // elements between two time steps of the sequence tensors
    };
    auto st = std::make_shared<State>(ctx);
    b200k_lstm_params& p = st->p;
    std::memset(&p, 0, sizeof(p));
    const TensorInfo& x = info.m_InputTensorInfos[0];
    const TensorInfo& h = info.m_InputTensorInfos[1];
    const TensorInfo& c = info.m_InputTensorInfos[2];
    p.output_size = static_cast<int32_t>(h.GetShape()[1]); p.num_units = static_cast<int32_t>(c.GetShape()[1]);
    if (sequence)
    {
        if (x.GetNumDimensions() != 3) { throw InvalidArgumentException("B200Acc: UnidirectionalSequenceLstm needs a 3-D input"); }
        const int64_t d0 = x.GetShape()[0], d1 = x.GetShape()[1];
        p.input_size = static_cast<int32_t>(x.GetShape()[2]);
        st->steps = prm.m_TimeMajor ? d0 : d1;
        p.batch = static_cast<int32_t>(prm.m_TimeMajor ? d1 : d0);
        // time major [T, B, I]: a step is a dense [B, I] block; batch major [B, T, I]: its rows are T * I apart
        p.input_stride = prm.m_TimeMajor ? p.input_size : st->steps * p.input_size;
        p.output_stride = prm.m_TimeMajor ? p.output_size : st->steps * p.output_size;
        st->stepIn = prm.m_TimeMajor ? static_cast<int64_t>(p.batch) * p.input_size : p.input_size;
        st->stepOut = prm.m_TimeMajor ? static_cast<int64_t>(p.batch) * p.output_size : p.output_size;
    }
    else
    {
        p.batch = static_cast<int32_t>(x.GetShape()[0]); p.input_size = static_cast<int32_t>(x.GetShape()[1]);
        p.input_stride = p.input_size; p.output_stride = p.output_size;
    }
    auto up = [&](const ConstTensorHandle* t) -> const float*
    {
        if (!t) { return nullptr; }
        return static_cast<const float*>(st->blobs.Upload(t->GetConstTensor<void>(), t->GetTensorInfo().GetNumBytes()));
    };
    if (!prm.m_CifgEnabled) { p.w_i2i = up(qd.m_InputToInputWeights); p.w_r2i = up(qd.m_RecurrentToInputWeights); p.b_i = up(qd.m_InputGateBias); }
    p.w_i2f = up(qd.m_InputToForgetWeights); p.w_i2c = up(qd.m_InputToCellWeights); p.w_i2o = up(qd.m_InputToOutputWeights);
    p.w_r2f = up(qd.m_RecurrentToForgetWeights); p.w_r2c = up(qd.m_RecurrentToCellWeights); p.w_r2o = up(qd.m_RecurrentToOutputWeights);
    p.b_f = up(qd.m_ForgetGateBias); p.b_c = up(qd.m_CellBias); p.b_o = up(qd.m_OutputGateBias);
    if (prm.m_PeepholeEnabled)
    {
        if (!prm.m_CifgEnabled) { p.w_c2i = up(qd.m_CellToInputWeights); }
        p.w_c2f = up(qd.m_CellToForgetWeights); p.w_c2o = up(qd.m_CellToOutputWeights);
    }
    if (prm.m_LayerNormEnabled)
    {
        if (!prm.m_CifgEnabled) { p.ln_i = up(qd.m_InputLayerNormWeights); }
        p.ln_f = up(qd.m_ForgetLayerNormWeights); p.ln_c = up(qd.m_CellLayerNormWeights); p.ln_o = up(qd.m_OutputLayerNormWeights);
    }
    if (prm.m_ProjectionEnabled) { p.w_proj = up(qd.m_ProjectionWeights); p.b_proj = up(qd.m_ProjectionBias); }
    p.activation = static_cast<int32_t>(prm.m_ActivationFunc);
    p.cell_clip = prm.m_ClippingThresCell; p.projection_clip = prm.m_ClippingThresProj;
    p.layer_norm_eps = 1e-8f;                                  // RefLstmWorkload.hpp: m_LayerNormEpsilon
    // outputs: Lstm: scratch, outputStateOut, cellStateOut, output; the sequence layer: outputStateOut, cellStateOut, output
    // (the reference's sequence workload leaves its two state outputs unwritten, RefUnidirectionalSequenceLstmWorkload.cpp:
    // 95-123; here they hold the running and finally the last states)
    const unsigned int o0 = sequence ? 0u : 1u;
    return Make<QD>(d, info, ctx, [st, o0](const QD& data, cudaStream_t s)
    {
        b200k_lstm_params q = st->p;
        const float* x0 = static_cast<const float*>(Dev(data.m_Inputs[0]));
        float* out0 = static_cast<float*>(Dev(data.m_Outputs[o0 + 2]));
        q.output_state_out = static_cast<float*>(Dev(data.m_Outputs[o0]));
        q.cell_state_out = static_cast<float*>(Dev(data.m_Outputs[o0 + 1]));
        for (int64_t t = 0; t < st->steps; ++t)
        {
            // the first step reads the state inputs, the others update the state outputs in place
            q.output_state_in = t == 0 ? static_cast<const float*>(Dev(data.m_Inputs[1])) : q.output_state_out;
            q.cell_state_in = t == 0 ? static_cast<const float*>(Dev(data.m_Inputs[2])) : q.cell_state_out;
            q.input = x0 + t * st->stepIn;
            q.output = out0 + t * st->stepOut;
            B200CheckStatus(b200k_lstm_step_f32(&q, s));
        }
    });
}

// Device copies of the QLstm weights: the descriptor's ConstTensorHandles are released by the layer right after
// CreateWorkload (src/armnn/LoadedNetwork.cpp:396), as RefQLstmWorkload's AssignScopedTensorHandle copies show.
std::unique_ptr<IWorkload> MakeQLstm(const QueueDescriptor& d, const WorkloadInfo& info, const ContextPtr& ctx)
{
    const auto& qd = *PolymorphicDowncast<const QLstmQueueDescriptor*>(&d);
    auto st = std::make_shared<SimpleState<b200k_qlstm_params>>(ctx);
    b200k_qlstm_params& p = st->p;
    std::memset(&p, 0, sizeof(p));
    const TensorInfo& x = info.m_InputTensorInfos[0];
    const TensorInfo& h = info.m_InputTensorInfos[1];
    const TensorInfo& c = info.m_InputTensorInfos[2];
    const TensorInfo& out = info.m_OutputTensorInfos[2];
    p.batch = x.GetShape()[0]; p.input_size = x.GetShape()[1];
    p.output_size = h.GetShape()[1]; p.num_units = c.GetShape()[1];
    p.input_scale = x.GetQuantizationScale(); p.input_zp = x.GetQuantizationOffset();
    p.output_state_scale = h.GetQuantizationScale(); p.output_state_zp = h.GetQuantizationOffset();
    p.cell_state_scale = c.GetQuantizationScale();
    p.output_scale = out.GetQuantizationScale(); p.output_zp = out.GetQuantizationOffset();
    const auto& prm = qd.m_Parameters;
    auto up = [&](const ConstTensorHandle* t, float* scale) -> const void*
    {
        if (!t) { return nullptr; }
        if (scale) { *scale = t->GetTensorInfo().GetQuantizationScale(); }
        return st->blobs.Upload(t->GetConstTensor<void>(), t->GetTensorInfo().GetNumBytes());
    };
    if (!prm.m_CifgEnabled)
    {
        p.w_i2i = static_cast<const int8_t*>(up(qd.m_InputToInputWeights, &p.s_i2i));
        p.w_r2i = static_cast<const int8_t*>(up(qd.m_RecurrentToInputWeights, &p.s_r2i));
    }
    p.w_i2f = static_cast<const int8_t*>(up(qd.m_InputToForgetWeights, &p.s_i2f));
    p.w_i2c = static_cast<const int8_t*>(up(qd.m_InputToCellWeights, &p.s_i2c));
    p.w_i2o = static_cast<const int8_t*>(up(qd.m_InputToOutputWeights, &p.s_i2o));
    p.w_r2f = static_cast<const int8_t*>(up(qd.m_RecurrentToForgetWeights, &p.s_r2f));
    p.w_r2c = static_cast<const int8_t*>(up(qd.m_RecurrentToCellWeights, &p.s_r2c));
    p.w_r2o = static_cast<const int8_t*>(up(qd.m_RecurrentToOutputWeights, &p.s_r2o));
    if (prm.m_PeepholeEnabled)
    {
        if (!prm.m_CifgEnabled) { p.w_c2i = static_cast<const int16_t*>(up(qd.m_CellToInputWeights, &p.s_c2i)); }
        p.w_c2f = static_cast<const int16_t*>(up(qd.m_CellToForgetWeights, &p.s_c2f));
        p.w_c2o = static_cast<const int16_t*>(up(qd.m_CellToOutputWeights, &p.s_c2o));
    }
    if (prm.m_LayerNormEnabled)
    {
        // gate biases are only read with layer norm, at scale (layer-norm weight scale / 1024)
        // (RefQLstmWorkload.cpp:261-287)
        if (!prm.m_CifgEnabled)
        {
            p.ln_i = static_cast<const int16_t*>(up(qd.m_InputLayerNormWeights, &p.s_lni));
            p.b_i = static_cast<const int32_t*>(up(qd.m_InputGateBias, nullptr));
            p.s_bi = p.s_lni / 1024;
        }
        p.ln_f = static_cast<const int16_t*>(up(qd.m_ForgetLayerNormWeights, &p.s_lnf));
        p.ln_c = static_cast<const int16_t*>(up(qd.m_CellLayerNormWeights, &p.s_lnc));
        p.ln_o = static_cast<const int16_t*>(up(qd.m_OutputLayerNormWeights, &p.s_lno));
        p.b_f = static_cast<const int32_t*>(up(qd.m_ForgetGateBias, nullptr)); p.s_bf = p.s_lnf / 1024;
        p.b_c = static_cast<const int32_t*>(up(qd.m_CellBias, nullptr));       p.s_bc = p.s_lnc / 1024;
        p.b_o = static_cast<const int32_t*>(up(qd.m_OutputGateBias, nullptr)); p.s_bo = p.s_lno / 1024;
    }
    if (prm.m_ProjectionEnabled)
    {
        p.w_proj = static_cast<const int8_t*>(up(qd.m_ProjectionWeights, &p.s_proj));
        p.b_proj = static_cast<const int32_t*>(up(qd.m_ProjectionBias, &p.s_bproj));
    }
    p.cell_clip = prm.m_CellClip; p.projection_clip = prm.m_ProjectionClip;
    p.input_intermediate_scale = prm.m_InputIntermediateScale;
    p.forget_intermediate_scale = prm.m_ForgetIntermediateScale;
    p.cell_intermediate_scale = prm.m_CellIntermediateScale;
    p.output_intermediate_scale = prm.m_OutputIntermediateScale;
    p.hidden_state_scale = prm.m_HiddenStateScale; p.hidden_state_zp = prm.m_HiddenStateZeroPoint;
    return Make<QLstmQueueDescriptor>(d, info, ctx, [st](const QLstmQueueDescriptor& data, cudaStream_t s)
    {
        b200k_qlstm_params& q = st->p;
        q.input = static_cast<const int8_t*>(Dev(data.m_Inputs[0]));
        q.output_state_in = static_cast<const int8_t*>(Dev(data.m_Inputs[1]));
        q.cell_state_in = static_cast<const int16_t*>(Dev(data.m_Inputs[2]));
        q.output_state_out = static_cast<int8_t*>(Dev(data.m_Outputs[0]));
        q.cell_state_out = static_cast<int16_t*>(Dev(data.m_Outputs[1]));
        q.output = static_cast<int8_t*>(Dev(data.m_Outputs[2]));
        B200CheckStatus(b200k_qlstm_step(&q, s));
    });
}

}  // namespace

B200WorkloadFactory::B200WorkloadFactory(const std::shared_ptr<B200Context>& ctx, const std::shared_ptr<B200MemoryManager>& memoryManager)
    : m_Ctx(ctx), m_MemoryManager(memoryManager) {}

const BackendId& B200WorkloadFactory::GetBackendId() const
{
    static const BackendId s_Id{B200BackendId()};
    return s_Id;
}

bool B200WorkloadFactory::IsLayerSupported(const IConnectableLayer& layer, Optional<DataType> dataType, std::string& reason)
{
    static const BackendId s_Id{B200BackendId()};
    return IWorkloadFactory::IsLayerSupported(s_Id, layer, dataType, reason);
}

std::unique_ptr<ITensorHandle> B200WorkloadFactory::CreateTensorHandle(const TensorInfo& info, const bool isMemoryManaged) const
{
    return std::make_unique<B200TensorHandle>(info, m_Ctx, isMemoryManaged ? m_MemoryManager : nullptr);
}

std::unique_ptr<ITensorHandle> B200WorkloadFactory::CreateTensorHandle(const TensorInfo& info, DataLayout, const bool isMemoryManaged) const
{
    return std::make_unique<B200TensorHandle>(info, m_Ctx, isMemoryManaged ? m_MemoryManager : nullptr);
}

std::unique_ptr<IWorkload> B200WorkloadFactory::CreateWorkload(LayerType type, const QueueDescriptor& d,
                                                               const WorkloadInfo& info) const
{
    const ContextPtr& ctx = m_Ctx;
    switch (type)
    {
        case LayerType::Input:
            return std::make_unique<CopyMemGenericWorkload>(*PolymorphicDowncast<const InputQueueDescriptor*>(&d), info);
        case LayerType::Output:
            return std::make_unique<CopyMemGenericWorkload>(*PolymorphicDowncast<const OutputQueueDescriptor*>(&d), info);
        case LayerType::MemCopy:
            return std::make_unique<CopyMemGenericWorkload>(*PolymorphicDowncast<const MemCopyQueueDescriptor*>(&d), info);
        case LayerType::MemImport:
            return std::make_unique<ImportMemGenericWorkload>(*PolymorphicDowncast<const MemImportQueueDescriptor*>(&d), info);
        case LayerType::Constant:
        {
            // One copy of the layer's blob into its output handle.  LoadedNetwork executes the Constant workloads at load
            // time (src/armnn/LoadedNetwork.cpp:565-568) and then again with every inference, as members of the workload
            // queue (LoadedNetwork.cpp:1267): like ClConstantWorkload (src/backends/cl/workloads/ClConstantWorkload.cpp:61)
            // only the first execution copies.
            auto ranOnce = std::make_shared<bool>(false);
            return Make<ConstantQueueDescriptor>(d, info, ctx, [ranOnce](const ConstantQueueDescriptor& data, cudaStream_t s)
            {
                if (*ranOnce) { return; }
                const ConstTensorHandle* src = data.m_LayerOutput;
                if (!src) { throw InvalidArgumentException("B200Acc: Constant workload without data"); }
                B200Check(cudaMemcpyAsync(Dev(data.m_Outputs[0]), src->GetConstTensor<void>(),
                                          src->GetTensorInfo().GetNumBytes(), cudaMemcpyHostToDevice, s), "cudaMemcpyAsync H2D");
                B200Check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
                *ranOnce = true;
            }, false);
        }
        case LayerType::Reshape:
        {
            const size_t bytes = info.m_InputTensorInfos[0].GetNumBytes();
            return Make<ReshapeQueueDescriptor>(d, info, ctx, [bytes](const ReshapeQueueDescriptor& data, cudaStream_t s)
            {
                B200Check(cudaMemcpyAsync(Dev(data.m_Outputs[0]), Dev(data.m_Inputs[0]), bytes, cudaMemcpyDeviceToDevice, s),
                          "cudaMemcpyAsync D2D");
            });
        }
        case LayerType::Convolution2d:
            return MakeConv<Convolution2dQueueDescriptor>(d, info, ctx, false);
        case LayerType::DepthwiseConvolution2d:
            return MakeConv<DepthwiseConvolution2dQueueDescriptor>(d, info, ctx, true);
        case LayerType::FullyConnected:
            return MakeFc(d, info, ctx);
        case LayerType::ElementwiseBinary:
        {
            const auto& qd = *PolymorphicDowncast<const ElementwiseBinaryQueueDescriptor*>(&d);
            return MakeEltwise(d, info, ctx, static_cast<int32_t>(qd.m_Parameters.m_Operation), qd.GetAdditionalInformation<ActivationDescriptor>());
        }
        case LayerType::Addition:
            return MakeEltwise(d, info, ctx, static_cast<int32_t>(BinaryOperation::Add), d.GetAdditionalInformation<ActivationDescriptor>());
        case LayerType::Multiplication:
            return MakeEltwise(d, info, ctx, static_cast<int32_t>(BinaryOperation::Mul), d.GetAdditionalInformation<ActivationDescriptor>());
        case LayerType::Subtraction:
            return MakeEltwise(d, info, ctx, static_cast<int32_t>(BinaryOperation::Sub), d.GetAdditionalInformation<ActivationDescriptor>());
        case LayerType::Division:
            return MakeEltwise(d, info, ctx, static_cast<int32_t>(BinaryOperation::Div), d.GetAdditionalInformation<ActivationDescriptor>());
        case LayerType::Maximum:
            return MakeEltwise(d, info, ctx, static_cast<int32_t>(BinaryOperation::Maximum), d.GetAdditionalInformation<ActivationDescriptor>());
        case LayerType::Minimum:
            return MakeEltwise(d, info, ctx, static_cast<int32_t>(BinaryOperation::Minimum), d.GetAdditionalInformation<ActivationDescriptor>());
        case LayerType::Prelu:
            return MakeEltwise(d, info, ctx, B200K_ELTWISE_PRELU, nullptr);
        case LayerType::Comparison:
            return MakeEltwise(d, info, ctx, 200 + static_cast<int32_t>(PolymorphicDowncast<const ComparisonQueueDescriptor*>(&d)->m_Parameters.m_Operation), nullptr);
        case LayerType::LogicalBinary:
            return MakeEltwise(d, info, ctx, 210 + static_cast<int32_t>(PolymorphicDowncast<const LogicalBinaryQueueDescriptor*>(&d)->m_Parameters.m_Operation), nullptr);
        case LayerType::Activation:
        {
            const auto& qd = *PolymorphicDowncast<const ActivationQueueDescriptor*>(&d);
            auto st = std::make_shared<SimpleState<b200k_activation_params>>(ctx);
            std::memset(&st->p, 0, sizeof(st->p));
            st->p.x = Operand(info.m_InputTensorInfos[0], st->blobs);
            st->p.y = Operand(info.m_OutputTensorInfos[0], st->blobs);
            st->p.count = info.m_InputTensorInfos[0].GetNumElements();
            st->p.function = static_cast<int32_t>(qd.m_Parameters.m_Function);
            st->p.a = qd.m_Parameters.m_A; st->p.b = qd.m_Parameters.m_B;
            return Make<ActivationQueueDescriptor>(d, info, ctx, [st](const ActivationQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_activation_q8(&st->p, s));
            });
        }
        case LayerType::Pooling2d:
        {
            const auto& qd = *PolymorphicDowncast<const Pooling2dQueueDescriptor*>(&d);
            const auto& q = qd.m_Parameters;
            auto st = std::make_shared<SimpleState<b200k_pool2d_params>>(ctx);
            b200k_pool2d_params& p = st->p;
            std::memset(&p, 0, sizeof(p));
            // an NCHW layer runs as re-layout -> NHWC kernel -> re-layout (see MakeConv)
            const bool nchw = q.m_DataLayout == DataLayout::NCHW;
            auto lay = std::make_shared<LayoutState>();
            TensorInfo x = info.m_InputTensorInfos[0], y = info.m_OutputTensorInfos[0];
            if (nchw)
            {
                lay->in = Relayout(x, kNchwToNhwc, st->blobs);
                lay->x = st->blobs.Alloc(x.GetNumBytes());
                x = NhwcOf(x);
                const TensorInfo yNhwc = NhwcOf(y);
                lay->out = Relayout(yNhwc, kNhwcToNchw, st->blobs);
                lay->y = st->blobs.Alloc(y.GetNumBytes());
                y = yNhwc;
            }
            p.x = Operand(x, st->blobs); p.y = Operand(y, st->blobs);
            p.n = x.GetShape()[0]; p.h = x.GetShape()[1]; p.wd = x.GetShape()[2]; p.c = x.GetShape()[3];
            p.oh = y.GetShape()[1]; p.ow = y.GetShape()[2];
            p.pool_h = q.m_PoolHeight; p.pool_w = q.m_PoolWidth; p.stride_h = q.m_StrideY; p.stride_w = q.m_StrideX;
            p.pad_top = q.m_PadTop; p.pad_bottom = q.m_PadBottom; p.pad_left = q.m_PadLeft; p.pad_right = q.m_PadRight;
            p.pool_type = static_cast<int32_t>(q.m_PoolType); p.padding_method = static_cast<int32_t>(q.m_PaddingMethod);
            return Make<Pooling2dQueueDescriptor>(d, info, ctx, [st, lay, nchw](const Pooling2dQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                if (nchw)
                {
                    lay->in.x.data = st->p.x.data; lay->in.y.data = lay->x;
                    B200CheckStatus(b200k_view_copy_q(&lay->in, s));
                    lay->out.x.data = lay->y; lay->out.y.data = st->p.y.data;
                    st->p.x.data = lay->x; st->p.y.data = lay->y;
                }
                B200CheckStatus(b200k_pool2d_q8(&st->p, s));
                if (nchw) { B200CheckStatus(b200k_view_copy_q(&lay->out, s)); }
            });
        }
        case LayerType::TransposeConvolution2d:
        {
            // weights [OC, KH, KW, C] and bias are constant members of the queue descriptor (not input tensors): one
            // upload at workload creation
            const auto& qd = *PolymorphicDowncast<const TransposeConvolution2dQueueDescriptor*>(&d);
            if (!qd.m_Weight) { throw InvalidArgumentException("B200Acc: TransposeConvolution2d needs constant weights"); }
            auto st = std::make_shared<SimpleState<b200k_conv2d_params>>(ctx);
            b200k_conv2d_params& p = st->p;
            std::memset(&p, 0, sizeof(p));
            // an NCHW layer runs as re-layout -> NHWC kernel -> re-layout (see MakeConv); its [O, I, H, W] weights are
            // re-ordered to [O, H, W, I] on the host before the upload
            const bool nchw = qd.m_Parameters.m_DataLayout == DataLayout::NCHW;
            auto lay = std::make_shared<LayoutState>();
            TensorInfo x = info.m_InputTensorInfos[0], y = info.m_OutputTensorInfos[0], w = qd.m_Weight->GetTensorInfo();
            std::vector<uint8_t> wHost(static_cast<const uint8_t*>(qd.m_Weight->GetConstTensor<void>()),
                                       static_cast<const uint8_t*>(qd.m_Weight->GetConstTensor<void>()) + w.GetNumBytes());
            if (nchw)
            {
                lay->in = Relayout(x, kNchwToNhwc, st->blobs);
                lay->x = st->blobs.Alloc(x.GetNumBytes());
                x = NhwcOf(x);
                const TensorInfo yNhwc = NhwcOf(y);
                lay->out = Relayout(yNhwc, kNhwcToNchw, st->blobs);
                lay->y = st->blobs.Alloc(y.GetNumBytes());
                y = yNhwc;
                const TensorShape ws = w.GetShape();                       // [O, I, H, W], one byte per element
                const std::vector<uint8_t> src = wHost;
                for (unsigned int o = 0; o < ws[0]; ++o) for (unsigned int i = 0; i < ws[1]; ++i)
                for (unsigned int hh = 0; hh < ws[2]; ++hh) for (unsigned int ww = 0; ww < ws[3]; ++ww)
                {
                    wHost[((static_cast<size_t>(o) * ws[2] + hh) * ws[3] + ww) * ws[1] + i] = src[((static_cast<size_t>(o) * ws[1] + i) * ws[2] + hh) * ws[3] + ww];
                }
                w = NhwcOf(w);
            }
            p.x = Operand(x, st->blobs); p.y = Operand(y, st->blobs); p.w = Operand(w, st->blobs);
            p.w.data = st->blobs.Upload(wHost.data(), wHost.size());
            if (qd.m_Parameters.m_BiasEnabled && qd.m_Bias)
            {
                const TensorInfo& b = qd.m_Bias->GetTensorInfo();
                p.bias = Operand(b, st->blobs);
                p.bias.data = st->blobs.Upload(qd.m_Bias->GetConstTensor<void>(), b.GetNumBytes());
            }
            p.n = x.GetShape()[0]; p.h = x.GetShape()[1]; p.wd = x.GetShape()[2]; p.c = x.GetShape()[3];
            p.oh = y.GetShape()[1]; p.ow = y.GetShape()[2]; p.oc = y.GetShape()[3];
            p.kh = w.GetShape()[1]; p.kw = w.GetShape()[2];
            if (w.GetShape()[0] != y.GetShape()[3] || w.GetShape()[3] != x.GetShape()[3]) { throw InvalidArgumentException("B200Acc: TransposeConvolution2d weights do not match the channel counts"); }
            p.stride_h = qd.m_Parameters.m_StrideY; p.stride_w = qd.m_Parameters.m_StrideX;
            p.pad_top = qd.m_Parameters.m_PadTop; p.pad_left = qd.m_Parameters.m_PadLeft;
            p.dil_h = p.dil_w = 1;
            Clamp(qd.GetAdditionalInformation<ActivationDescriptor>(), y, p.clamp_lo, p.clamp_hi);
            return Make<TransposeConvolution2dQueueDescriptor>(d, info, ctx, [st, lay, nchw](const TransposeConvolution2dQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                if (nchw)
                {
                    lay->in.x.data = st->p.x.data; lay->in.y.data = lay->x;
                    B200CheckStatus(b200k_view_copy_q(&lay->in, s));
                    lay->out.x.data = lay->y; lay->out.y.data = st->p.y.data;
                    st->p.x.data = lay->x; st->p.y.data = lay->y;
                }
                B200CheckStatus(b200k_transpose_conv2d_q8(&st->p, s));
                if (nchw) { B200CheckStatus(b200k_view_copy_q(&lay->out, s)); }
            });
        }
        case LayerType::ElementwiseUnary:
        {
            const auto& qd = *PolymorphicDowncast<const ElementwiseUnaryQueueDescriptor*>(&d);
            auto st = std::make_shared<SimpleState<b200k_unary_params>>(ctx);
            b200k_unary_params& p = st->p;
            std::memset(&p, 0, sizeof(p));
            const TensorInfo& x = info.m_InputTensorInfos[0];
            p.x = Operand(x, st->blobs); p.y = Operand(info.m_OutputTensorInfos[0], st->blobs);
            p.count = static_cast<int64_t>(x.GetNumElements());
            p.operation = static_cast<int32_t>(qd.m_Parameters.m_Operation);
            return Make<ElementwiseUnaryQueueDescriptor>(d, info, ctx, [st](const ElementwiseUnaryQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_unary_q(&st->p, s));
            });
        }
        case LayerType::Reduce:
        {
            const auto& qd = *PolymorphicDowncast<const ReduceQueueDescriptor*>(&d);
            return MakeReduce<ReduceQueueDescriptor>(d, info, ctx, qd.m_Parameters.m_vAxis, static_cast<int32_t>(qd.m_Parameters.m_ReduceOperation));
        }
        case LayerType::Mean:
        {
            const auto& axes = PolymorphicDowncast<const MeanQueueDescriptor*>(&d)->m_Parameters.m_Axis;
            if (info.m_InputTensorInfos[0].GetNumDimensions() != 4 || axes != std::vector<unsigned int>{1, 2})
            {
                // RefMeanWorkload is armnn::Reduce with ReduceOperation::Mean (RefMeanWorkload.cpp)
                return MakeReduce<MeanQueueDescriptor>(d, info, ctx, axes, 2);
            }
            auto st = std::make_shared<SimpleState<b200k_mean_params>>(ctx);
            b200k_mean_params& p = st->p;
            std::memset(&p, 0, sizeof(p));
            const TensorInfo& x = info.m_InputTensorInfos[0];
            p.x = Operand(x, st->blobs); p.y = Operand(info.m_OutputTensorInfos[0], st->blobs);
            p.n = x.GetShape()[0]; p.h = x.GetShape()[1]; p.wd = x.GetShape()[2]; p.c = x.GetShape()[3];
            return Make<MeanQueueDescriptor>(d, info, ctx, [st](const MeanQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_mean_hw_q8(&st->p, s));
            });
        }
        case LayerType::Softmax:
        {
            const auto& qd = *PolymorphicDowncast<const SoftmaxQueueDescriptor*>(&d);
            auto st = std::make_shared<SimpleState<b200k_softmax_params>>(ctx);
            b200k_softmax_params& p = st->p;
            std::memset(&p, 0, sizeof(p));
            const TensorInfo& x = info.m_InputTensorInfos[0];
            p.x = Operand(x, st->blobs); p.y = Operand(info.m_OutputTensorInfos[0], st->blobs);
            const int rank = static_cast<int>(x.GetNumDimensions());
            int axis = qd.m_Parameters.m_Axis < 0 ? rank + qd.m_Parameters.m_Axis : qd.m_Parameters.m_Axis;
            p.outer = 1; p.inner = 1;
            for (int i = 0; i < axis; ++i) { p.outer *= x.GetShape()[i]; }
            for (int i = axis + 1; i < rank; ++i) { p.inner *= x.GetShape()[i]; }
            p.axis_size = x.GetShape()[axis];
            p.beta = qd.m_Parameters.m_Beta;
            return Make<SoftmaxQueueDescriptor>(d, info, ctx, [st](const SoftmaxQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_softmax_q8(&st->p, s));
            });
        }
        case LayerType::Gather:
        {
            const auto& qd = *PolymorphicDowncast<const GatherQueueDescriptor*>(&d);
            auto st = std::make_shared<SimpleState<b200k_gather_params>>(ctx);
            std::memset(&st->p, 0, sizeof(st->p));
            st->p.x = Operand(info.m_InputTensorInfos[0], st->blobs); st->p.y = Operand(info.m_OutputTensorInfos[0], st->blobs);
            RowsOf(info.m_InputTensorInfos[0].GetShape(), qd.m_Parameters.m_Axis, st->p.outer, st->p.axis_size, st->p.inner);
            st->p.n_indices = static_cast<int32_t>(info.m_InputTensorInfos[1].GetNumElements());
            if (info.m_OutputTensorInfos[0].GetNumElements() !=
                static_cast<unsigned int>(st->p.outer) * static_cast<unsigned int>(st->p.n_indices) * static_cast<unsigned int>(st->p.inner))
            {
                throw InvalidArgumentException("B200Acc: Gather output shape does not match the gathered input");
            }
            return Make<GatherQueueDescriptor>(d, info, ctx, [st](const GatherQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.indices = static_cast<const int32_t*>(Dev(data.m_Inputs[1]));
                st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_gather_q(&st->p, s));
            });
        }
        case LayerType::ScatterNd:
        {
            const auto& prm = PolymorphicDowncast<const ScatterNdQueueDescriptor*>(&d)->m_Parameters;
            auto st = std::make_shared<SimpleState<b200k_scatter_nd_params>>(ctx);
            b200k_scatter_nd_params& p = st->p;
            std::memset(&p, 0, sizeof(p));
            const TensorInfo& idx = info.m_InputTensorInfos[1];
            const TensorInfo& y = info.m_OutputTensorInfos[0];
            if (prm.m_AxisEnabled || idx.GetNumDimensions() != 2) { throw InvalidArgumentException("B200Acc: ScatterNd without axis, indices [n, nd]"); }
            const bool withInput = prm.m_InputEnabled;
            if (withInput) { p.x = Operand(info.m_InputTensorInfos[0], st->blobs); }
            p.updates = Operand(info.m_InputTensorInfos[2], st->blobs); p.y = Operand(y, st->blobs);
            p.n_indices = static_cast<int32_t>(idx.GetShape()[0]); p.nd = static_cast<int32_t>(idx.GetShape()[1]);
            if (p.nd < 1 || p.nd > 8 || static_cast<unsigned int>(p.nd) > y.GetNumDimensions()) { throw InvalidArgumentException("B200Acc: ScatterNd index tuples do not fit the output"); }
            p.inner = 1;
            for (unsigned int i = 0; i < y.GetNumDimensions(); ++i)
            {
                if (i < static_cast<unsigned int>(p.nd)) { p.dims[i] = static_cast<int32_t>(y.GetShape()[i]); } else { p.inner *= static_cast<int32_t>(y.GetShape()[i]); }
            }
            if (info.m_InputTensorInfos[2].GetNumElements() != static_cast<unsigned int>(p.n_indices) * static_cast<unsigned int>(p.inner))
            {
                throw InvalidArgumentException("B200Acc: ScatterNd updates do not match the index tuples");
            }
            p.function = static_cast<int32_t>(prm.m_Function);
            return Make<ScatterNdQueueDescriptor>(d, info, ctx, [st, withInput](const ScatterNdQueueDescriptor& data, cudaStream_t s)
            {
                if (withInput) { st->p.x.data = Dev(data.m_Inputs[0]); }
                st->p.indices = static_cast<const int32_t*>(Dev(data.m_Inputs[1]));
                st->p.updates.data = Dev(data.m_Inputs[2]); st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_scatter_nd_q(&st->p, s));
            });
        }
        case LayerType::ReverseV2:
        {
            auto st = std::make_shared<SimpleState<b200k_reverse_params>>(ctx);
            b200k_reverse_params& p = st->p;
            std::memset(&p, 0, sizeof(p));
            const TensorInfo& x = info.m_InputTensorInfos[0];
            if (x.GetNumDimensions() > 6) { throw InvalidArgumentException("B200Acc: ReverseV2 takes at most 6 dimensions"); }
            p.x = Operand(x, st->blobs); p.y = Operand(info.m_OutputTensorInfos[0], st->blobs);
            p.n_axes = static_cast<int32_t>(info.m_InputTensorInfos[1].GetNumElements());
            p.rank = static_cast<int32_t>(x.GetNumDimensions());
            for (unsigned int i = 0; i < x.GetNumDimensions(); ++i) { p.shape[i] = static_cast<int32_t>(x.GetShape()[i]); }
            return Make<ReverseV2QueueDescriptor>(d, info, ctx, [st](const ReverseV2QueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.axes = static_cast<const int32_t*>(Dev(data.m_Inputs[1]));
                st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_reverse_q(&st->p, s));
            });
        }
        case LayerType::GatherNd:
        {
            auto st = std::make_shared<SimpleState<b200k_gather_nd_params>>(ctx);
            b200k_gather_nd_params& p = st->p;
            std::memset(&p, 0, sizeof(p));
            const TensorInfo& x = info.m_InputTensorInfos[0];
            const TensorInfo& idx = info.m_InputTensorInfos[1];
            p.x = Operand(x, st->blobs); p.y = Operand(info.m_OutputTensorInfos[0], st->blobs);
            const unsigned int nd = idx.GetShape()[idx.GetNumDimensions() - 1];
            if (nd < 1 || nd > 8 || nd > x.GetNumDimensions()) { throw InvalidArgumentException("B200Acc: GatherNd index tuples do not fit the tensor"); }
            p.nd = static_cast<int32_t>(nd);
            p.n_indices = static_cast<int32_t>(idx.GetNumElements() / nd);
            p.inner = 1;
            for (unsigned int i = 0; i < x.GetNumDimensions(); ++i)
            {
                if (i < nd) { p.dims[i] = static_cast<int32_t>(x.GetShape()[i]); } else { p.inner *= static_cast<int32_t>(x.GetShape()[i]); }
            }
            if (info.m_OutputTensorInfos[0].GetNumElements() != static_cast<unsigned int>(p.n_indices) * static_cast<unsigned int>(p.inner))
            {
                throw InvalidArgumentException("B200Acc: GatherNd output shape does not match the gathered slices");
            }
            return Make<GatherNdQueueDescriptor>(d, info, ctx, [st](const GatherNdQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.indices = static_cast<const int32_t*>(Dev(data.m_Inputs[1]));
                st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_gather_nd_q(&st->p, s));
            });
        }
        case LayerType::BatchNormalization:
        {
            // the descriptor's constant handles are only valid during workload creation: the workload owns device copies
            const auto& qd = *PolymorphicDowncast<const BatchNormalizationQueueDescriptor*>(&d);
            auto st = std::make_shared<SimpleState<b200k_batch_norm_params>>(ctx);
            b200k_batch_norm_params& p = st->p;
            std::memset(&p, 0, sizeof(p));
            const TensorInfo& x = info.m_InputTensorInfos[0];
            if (x.GetNumDimensions() != 4 || !qd.m_Mean || !qd.m_Variance || !qd.m_Beta || !qd.m_Gamma) { throw InvalidArgumentException("B200Acc: BatchNormalization needs a 4-D input and four parameter tensors"); }
            p.x = Operand(x, st->blobs); p.y = Operand(info.m_OutputTensorInfos[0], st->blobs);
            p.nchw = qd.m_Parameters.m_DataLayout == DataLayout::NCHW ? 1 : 0;
            p.n = static_cast<int32_t>(x.GetShape()[0]);
            p.c = static_cast<int32_t>(p.nchw ? x.GetShape()[1] : x.GetShape()[3]);
            p.hw = p.nchw ? static_cast<int64_t>(x.GetShape()[2]) * x.GetShape()[3] : static_cast<int64_t>(x.GetShape()[1]) * x.GetShape()[2];
            p.eps = qd.m_Parameters.m_Eps;
            auto constant = [&](const ConstTensorHandle* t)
            {
                if (t->GetTensorInfo().GetNumElements() != static_cast<unsigned int>(p.c)) { throw InvalidArgumentException("B200Acc: BatchNormalization parameters must hold one value per channel"); }
                b200k_qtensor q = Operand(t->GetTensorInfo(), st->blobs);
                q.data = st->blobs.Upload(t->GetConstTensor<void>(), t->GetTensorInfo().GetNumBytes());
                return q;
            };
            p.mean = constant(qd.m_Mean); p.variance = constant(qd.m_Variance); p.beta = constant(qd.m_Beta); p.gamma = constant(qd.m_Gamma);
            p.scratch = st->blobs.Alloc(2 * static_cast<size_t>(p.c) * sizeof(float));
            return Make<BatchNormalizationQueueDescriptor>(d, info, ctx, [st](const BatchNormalizationQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_batch_norm_q(&st->p, s));
            });
        }
        case LayerType::Normalization:
        {
            // the reference encodes the output with the input's TensorInfo (RefNormalizationWorkload.cpp:176-177) and its
            // Within variant reads the shape as [N, C, H, W] whatever the layout says (lines 25-28): both kept
            const auto& qd = *PolymorphicDowncast<const NormalizationQueueDescriptor*>(&d);
            auto st = std::make_shared<SimpleState<b200k_normalization_params>>(ctx);
            b200k_normalization_params& p = st->p;
            std::memset(&p, 0, sizeof(p));
            const TensorInfo& x = info.m_InputTensorInfos[0];
            if (x.GetNumDimensions() != 4 || qd.m_Parameters.m_NormMethodType != NormalizationAlgorithmMethod::LocalBrightness) { throw InvalidArgumentException("B200Acc: Normalization needs a 4-D input and the LocalBrightness method"); }
            p.x = Operand(x, st->blobs); p.y = Operand(x, st->blobs);
            p.channel_type = qd.m_Parameters.m_NormChannelType == NormalizationAlgorithmChannel::Within ? 1 : 0;
            const TensorShape& s = x.GetShape();
            p.n = static_cast<int32_t>(s[0]);
            if (p.channel_type == 1 || qd.m_Parameters.m_DataLayout == DataLayout::NCHW)
            {
                p.c = static_cast<int32_t>(s[1]); p.h = static_cast<int32_t>(s[2]); p.w = static_cast<int32_t>(s[3]); p.nchw = 1;
            }
            else
            {
                p.h = static_cast<int32_t>(s[1]); p.w = static_cast<int32_t>(s[2]); p.c = static_cast<int32_t>(s[3]); p.nchw = 0;
            }
            p.norm_size = qd.m_Parameters.m_NormSize;
            p.alpha = qd.m_Parameters.m_Alpha; p.beta = qd.m_Parameters.m_Beta; p.kappa = qd.m_Parameters.m_K;
            return Make<NormalizationQueueDescriptor>(d, info, ctx, [st](const NormalizationQueueDescriptor& data, cudaStream_t s2)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_normalization_q(&st->p, s2));
            });
        }
        case LayerType::InstanceNormalization:
        {
            const auto& qd = *PolymorphicDowncast<const InstanceNormalizationQueueDescriptor*>(&d);
            auto st = std::make_shared<SimpleState<b200k_instance_norm_params>>(ctx);
            b200k_instance_norm_params& p = st->p;
            std::memset(&p, 0, sizeof(p));
            const TensorInfo& x = info.m_InputTensorInfos[0];
            if (x.GetNumDimensions() != 4) { throw InvalidArgumentException("B200Acc: InstanceNormalization needs a 4-D input"); }
            p.x = Operand(x, st->blobs); p.y = Operand(info.m_OutputTensorInfos[0], st->blobs);
            p.nchw = qd.m_Parameters.m_DataLayout == DataLayout::NCHW ? 1 : 0;
            p.n = static_cast<int32_t>(x.GetShape()[0]);
            p.c = static_cast<int32_t>(p.nchw ? x.GetShape()[1] : x.GetShape()[3]);
            p.hw = p.nchw ? static_cast<int64_t>(x.GetShape()[2]) * x.GetShape()[3] : static_cast<int64_t>(x.GetShape()[1]) * x.GetShape()[2];
            p.gamma = qd.m_Parameters.m_Gamma; p.beta = qd.m_Parameters.m_Beta; p.eps = qd.m_Parameters.m_Eps;
            return Make<InstanceNormalizationQueueDescriptor>(d, info, ctx, [st](const InstanceNormalizationQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_instance_norm_q(&st->p, s));
            });
        }
        case LayerType::Convolution3d:
        {
            const auto& qd = *PolymorphicDowncast<const Convolution3dQueueDescriptor*>(&d);
            const auto& prm = qd.m_Parameters;
            auto st = std::make_shared<SimpleState<b200k_conv3d_params>>(ctx);
            b200k_conv3d_params& p = st->p;
            std::memset(&p, 0, sizeof(p));
            const TensorInfo& x = info.m_InputTensorInfos[0];
            const TensorInfo& w = info.m_InputTensorInfos[1];
            const TensorInfo& y = info.m_OutputTensorInfos[0];
            if (prm.m_DataLayout != DataLayout::NDHWC || x.GetNumDimensions() != 5 || w.GetNumDimensions() != 5 || y.GetNumDimensions() != 5)
            {
                throw InvalidArgumentException("B200Acc: Convolution3d needs 5-D NDHWC tensors");
            }
            p.x = Operand(x, st->blobs); p.w = Operand(w, st->blobs); p.y = Operand(y, st->blobs);
            const bool bias = prm.m_BiasEnabled && info.m_InputTensorInfos.size() > 2;
            if (bias) { p.bias = Operand(info.m_InputTensorInfos[2], st->blobs); }
            p.n = static_cast<int32_t>(x.GetShape()[0]); p.d = static_cast<int32_t>(x.GetShape()[1]); p.h = static_cast<int32_t>(x.GetShape()[2]);
            p.wd = static_cast<int32_t>(x.GetShape()[3]); p.c = static_cast<int32_t>(x.GetShape()[4]);
            p.od = static_cast<int32_t>(y.GetShape()[1]); p.oh = static_cast<int32_t>(y.GetShape()[2]); p.ow = static_cast<int32_t>(y.GetShape()[3]);
            p.oc = static_cast<int32_t>(y.GetShape()[4]);
            p.kd = static_cast<int32_t>(w.GetShape()[0]); p.kh = static_cast<int32_t>(w.GetShape()[1]); p.kw = static_cast<int32_t>(w.GetShape()[2]);
            if (w.GetShape()[3] != x.GetShape()[4] || w.GetShape()[4] != y.GetShape()[4]) { throw InvalidArgumentException("B200Acc: Convolution3d weights do not match the channel counts"); }
            p.stride_d = static_cast<int32_t>(prm.m_StrideZ); p.stride_h = static_cast<int32_t>(prm.m_StrideY); p.stride_w = static_cast<int32_t>(prm.m_StrideX);
            p.pad_front = static_cast<int32_t>(prm.m_PadFront); p.pad_top = static_cast<int32_t>(prm.m_PadTop); p.pad_left = static_cast<int32_t>(prm.m_PadLeft);
            p.dil_d = static_cast<int32_t>(prm.m_DilationZ); p.dil_h = static_cast<int32_t>(prm.m_DilationY); p.dil_w = static_cast<int32_t>(prm.m_DilationX);
            if (y.GetDataType() != DataType::Float32) { Clamp(qd.GetAdditionalInformation<ActivationDescriptor>(), y, p.clamp_lo, p.clamp_hi); }
            return Make<Convolution3dQueueDescriptor>(d, info, ctx, [st, bias](const Convolution3dQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.w.data = Dev(data.m_Inputs[1]);
                if (bias) { st->p.bias.data = Dev(data.m_Inputs[2]); }
                st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_conv3d_q(&st->p, s));
            });
        }
        case LayerType::Pooling3d:
        {
            const auto& prm = PolymorphicDowncast<const Pooling3dQueueDescriptor*>(&d)->m_Parameters;
            auto st = std::make_shared<SimpleState<b200k_pool3d_params>>(ctx);
            b200k_pool3d_params& p = st->p;
            std::memset(&p, 0, sizeof(p));
            const TensorInfo& x = info.m_InputTensorInfos[0];
            const TensorInfo& y = info.m_OutputTensorInfos[0];
            if (prm.m_DataLayout != DataLayout::NDHWC || x.GetNumDimensions() != 5 || y.GetNumDimensions() != 5) { throw InvalidArgumentException("B200Acc: Pooling3d needs 5-D NDHWC tensors"); }
            p.x = Operand(x, st->blobs); p.y = Operand(y, st->blobs);
            p.n = static_cast<int32_t>(x.GetShape()[0]); p.d = static_cast<int32_t>(x.GetShape()[1]); p.h = static_cast<int32_t>(x.GetShape()[2]);
            p.wd = static_cast<int32_t>(x.GetShape()[3]); p.c = static_cast<int32_t>(x.GetShape()[4]);
            p.od = static_cast<int32_t>(y.GetShape()[1]); p.oh = static_cast<int32_t>(y.GetShape()[2]); p.ow = static_cast<int32_t>(y.GetShape()[3]);
            p.pool_d = static_cast<int32_t>(prm.m_PoolDepth); p.pool_h = static_cast<int32_t>(prm.m_PoolHeight); p.pool_w = static_cast<int32_t>(prm.m_PoolWidth);
            p.stride_d = static_cast<int32_t>(prm.m_StrideZ); p.stride_h = static_cast<int32_t>(prm.m_StrideY); p.stride_w = static_cast<int32_t>(prm.m_StrideX);
            p.pad_front = static_cast<int32_t>(prm.m_PadFront); p.pad_back = static_cast<int32_t>(prm.m_PadBack); p.pad_top = static_cast<int32_t>(prm.m_PadTop);
            p.pad_bottom = static_cast<int32_t>(prm.m_PadBottom); p.pad_left = static_cast<int32_t>(prm.m_PadLeft); p.pad_right = static_cast<int32_t>(prm.m_PadRight);
            p.pool_type = static_cast<int32_t>(prm.m_PoolType);
            p.padding_method = prm.m_PaddingMethod == PaddingMethod::Exclude ? 1 : 0;
            return Make<Pooling3dQueueDescriptor>(d, info, ctx, [st](const Pooling3dQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_pool3d_q(&st->p, s));
            });
        }
        case LayerType::Shape:
        case LayerType::Rank:
        {
            // known when the network is loaded (RefShapeWorkload.hpp, RefRankWorkload.hpp write it at every execution):
            // a device constant copied into the output tensor
            auto st = std::make_shared<ViewState>(ctx);
            const TensorInfo& in = info.m_InputTensorInfos[0];
            const TensorInfo& out = info.m_OutputTensorInfos[0];
            std::vector<int32_t> values;
            if (type == LayerType::Shape) { for (unsigned int i = 0; i < in.GetNumDimensions(); ++i) { values.push_back(static_cast<int32_t>(in.GetShape()[i])); } }
            else { values.push_back(static_cast<int32_t>(in.GetNumDimensions())); }
            if (out.GetDataType() != DataType::Signed32 || out.GetNumElements() != values.size()) { throw InvalidArgumentException("B200Acc: Shape / Rank need a Signed32 output of the right size"); }
            ViewOp op = NewViewOp(out, out, st->blobs, 0, 0, 1);
            op.fixedSrc = st->blobs.Upload(values.data(), values.size() * sizeof(int32_t));
            op.p.shape[0] = static_cast<int32_t>(values.size()); op.p.src_strides[0] = 1; op.p.dst_strides[0] = 1;
            st->ops.push_back(op);
            if (type == LayerType::Shape) { return MakeViews<ShapeQueueDescriptor>(d, info, ctx, st); }
            return MakeViews<RankQueueDescriptor>(d, info, ctx, st);
        }
        case LayerType::FakeQuantization:
        {
            const auto& prm = PolymorphicDowncast<const FakeQuantizationQueueDescriptor*>(&d)->m_Parameters;
            auto st = std::make_shared<SimpleState<b200k_activation_params>>(ctx);
            std::memset(&st->p, 0, sizeof(st->p));
            st->p.x = Operand(info.m_InputTensorInfos[0], st->blobs); st->p.y = Operand(info.m_OutputTensorInfos[0], st->blobs);
            st->p.count = info.m_InputTensorInfos[0].GetNumElements();
            st->p.function = B200K_ACTIVATION_FAKE_QUANTIZATION; st->p.a = prm.m_Min; st->p.b = prm.m_Max;
            return Make<FakeQuantizationQueueDescriptor>(d, info, ctx, [st](const FakeQuantizationQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_activation_q8(&st->p, s));
            });
        }
        case LayerType::ConvertFp16ToFp32:
        case LayerType::ConvertFp32ToFp16:
        {
            auto st = std::make_shared<SimpleState<b200k_convert_fp16_params>>(ctx);
            std::memset(&st->p, 0, sizeof(st->p));
            st->p.count = info.m_InputTensorInfos[0].GetNumElements();
            st->p.to_half = type == LayerType::ConvertFp32ToFp16 ? 1 : 0;
            auto fn = [st](const QueueDescriptor& data, cudaStream_t s)
            {
                st->p.x = Dev(data.m_Inputs[0]); st->p.y = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_convert_fp16(&st->p, s));
            };
            if (type == LayerType::ConvertFp32ToFp16) { return Make<ConvertFp32ToFp16QueueDescriptor>(d, info, ctx, fn); }
            return Make<ConvertFp16ToFp32QueueDescriptor>(d, info, ctx, fn);
        }
        case LayerType::Cast:
        {
            auto st = std::make_shared<SimpleState<b200k_convert_params>>(ctx);
            std::memset(&st->p, 0, sizeof(st->p));
            st->p.x = Operand(info.m_InputTensorInfos[0], st->blobs);
            st->p.y = Operand(info.m_OutputTensorInfos[0], st->blobs);
            st->p.count = info.m_InputTensorInfos[0].GetNumElements();
            return Make<CastQueueDescriptor>(d, info, ctx, [st](const CastQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_cast_q(&st->p, s));
            });
        }
        case LayerType::Fill:
        {
            // every element of the output <- one element holding the value in the output's type (workloads/Fill.cpp:13-23)
            const auto& qd = *PolymorphicDowncast<const FillQueueDescriptor*>(&d);
            auto st = std::make_shared<ViewState>(ctx);
            const TensorInfo& out = info.m_OutputTensorInfos[0];
            const unsigned int rank = out.GetNumDimensions();
            if (rank < 1 || rank > 6) { throw InvalidArgumentException("B200Acc: Fill needs an output of 1 to 6 dimensions"); }
            uint8_t bytes[4];
            if (out.GetDataType() == DataType::Signed32) { const int32_t v = static_cast<int32_t>(qd.m_Parameters.m_Value); std::memcpy(bytes, &v, 4); }
            else { const float v = qd.m_Parameters.m_Value; std::memcpy(bytes, &v, 4); }
            ViewOp op = NewViewOp(out, out, st->blobs, 0, 0, rank);
            op.fixedSrc = st->blobs.Upload(bytes, sizeof(bytes));
            DenseStrides(out.GetShape(), op.p.dst_strides);
            for (unsigned int i = 0; i < rank; ++i) { op.p.shape[i] = static_cast<int32_t>(out.GetShape()[i]); }
            st->ops.push_back(op);
            return MakeViews<FillQueueDescriptor>(d, info, ctx, st);
        }
        case LayerType::Floor:
        {
            auto st = std::make_shared<SimpleState<b200k_unary_params>>(ctx);
            std::memset(&st->p, 0, sizeof(st->p));
            st->p.x = Operand(info.m_InputTensorInfos[0], st->blobs); st->p.y = Operand(info.m_OutputTensorInfos[0], st->blobs);
            st->p.count = info.m_InputTensorInfos[0].GetNumElements();
            st->p.operation = 9;
            return Make<FloorQueueDescriptor>(d, info, ctx, [st](const FloorQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_unary_q(&st->p, s));
            });
        }
        case LayerType::LogSoftmax:
        {
            const auto& qd = *PolymorphicDowncast<const LogSoftmaxQueueDescriptor*>(&d);
            auto st = std::make_shared<SimpleState<b200k_softmax_params>>(ctx);
            std::memset(&st->p, 0, sizeof(st->p));
            st->p.x = Operand(info.m_InputTensorInfos[0], st->blobs); st->p.y = Operand(info.m_OutputTensorInfos[0], st->blobs);
            RowsOf(info.m_InputTensorInfos[0].GetShape(), qd.m_Parameters.m_Axis, st->p.outer, st->p.axis_size, st->p.inner);
            st->p.beta = qd.m_Parameters.m_Beta;
            return Make<LogSoftmaxQueueDescriptor>(d, info, ctx, [st](const LogSoftmaxQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_log_softmax_q(&st->p, s));
            });
        }
        case LayerType::L2Normalization:
        {
            // the channel dimension of the shape padded to four dimensions with leading 1s
            // (RefL2NormalizationWorkload.cpp:41-71); without one, every element is its own channel
            const auto& qd = *PolymorphicDowncast<const L2NormalizationQueueDescriptor*>(&d);
            auto st = std::make_shared<SimpleState<b200k_softmax_params>>(ctx);
            std::memset(&st->p, 0, sizeof(st->p));
            const TensorInfo& x = info.m_InputTensorInfos[0];
            st->p.x = Operand(x, st->blobs); st->p.y = Operand(info.m_OutputTensorInfos[0], st->blobs);
            const int rank = static_cast<int>(x.GetNumDimensions());
            const int axis = (qd.m_Parameters.m_DataLayout == DataLayout::NCHW ? 1 : 3) - (4 - rank);
            if (rank > 4) { throw InvalidArgumentException("B200Acc: L2Normalization takes at most 4 dimensions"); }
            if (axis < 0) { st->p.outer = static_cast<int32_t>(x.GetNumElements()); st->p.axis_size = 1; st->p.inner = 1; }
            else { RowsOf(x.GetShape(), axis, st->p.outer, st->p.axis_size, st->p.inner); }
            st->p.beta = qd.m_Parameters.m_Eps;
            return Make<L2NormalizationQueueDescriptor>(d, info, ctx, [st](const L2NormalizationQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_l2_normalization_q(&st->p, s));
            });
        }
        case LayerType::ArgMinMax:
        {
            const auto& qd = *PolymorphicDowncast<const ArgMinMaxQueueDescriptor*>(&d);
            auto st = std::make_shared<SimpleState<b200k_arg_min_max_params>>(ctx);
            std::memset(&st->p, 0, sizeof(st->p));
            st->p.x = Operand(info.m_InputTensorInfos[0], st->blobs);
            RowsOf(info.m_InputTensorInfos[0].GetShape(), qd.m_Parameters.m_Axis, st->p.outer, st->p.axis_size, st->p.inner);
            st->p.function = qd.m_Parameters.m_Function == ArgMinMaxFunction::Max ? 1 : 0;
            st->p.out_int64 = info.m_OutputTensorInfos[0].GetDataType() == DataType::Signed64 ? 1 : 0;
            if (info.m_OutputTensorInfos[0].GetNumElements() != static_cast<unsigned int>(st->p.outer) * static_cast<unsigned int>(st->p.inner))
            {
                throw InvalidArgumentException("B200Acc: ArgMinMax output shape does not drop the axis");
            }
            return Make<ArgMinMaxQueueDescriptor>(d, info, ctx, [st](const ArgMinMaxQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_arg_min_max_q(&st->p, s));
            });
        }
        case LayerType::Quantize:
        case LayerType::Dequantize:
        {
            auto st = std::make_shared<SimpleState<b200k_convert_params>>(ctx);
            std::memset(&st->p, 0, sizeof(st->p));
            st->p.x = Operand(info.m_InputTensorInfos[0], st->blobs);
            st->p.y = Operand(info.m_OutputTensorInfos[0], st->blobs);
            st->p.count = info.m_InputTensorInfos[0].GetNumElements();
            auto fn = [st](const QueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_convert_q(&st->p, s));
            };
            if (type == LayerType::Quantize) { return Make<QuantizeQueueDescriptor>(d, info, ctx, fn); }
            return Make<DequantizeQueueDescriptor>(d, info, ctx, fn);
        }
        case LayerType::BatchMatMul:
        {
            const auto& qd = *PolymorphicDowncast<const BatchMatMulQueueDescriptor*>(&d);
            auto st = std::make_shared<SimpleState<b200k_bmm_params>>(ctx);
            b200k_bmm_params& p = st->p;
            std::memset(&p, 0, sizeof(p));
            const TensorInfo& x = info.m_InputTensorInfos[0];
            const TensorInfo& y = info.m_InputTensorInfos[1];
            const TensorInfo& o = info.m_OutputTensorInfos[0];
            p.x = Operand(x, st->blobs); p.y = Operand(y, st->blobs); p.out = Operand(o, st->blobs);
            const unsigned ro = o.GetNumDimensions(), rx = x.GetNumDimensions(), ry = y.GetNumDimensions();
            p.m = o.GetShape()[ro - 2]; p.n = o.GetShape()[ro - 1];
            p.transpose_x = qd.m_Parameters.m_TransposeX; p.transpose_y = qd.m_Parameters.m_TransposeY;
            p.k = p.transpose_x ? x.GetShape()[rx - 2] : x.GetShape()[rx - 1];
            p.batch = static_cast<int32_t>(o.GetNumElements() / (static_cast<unsigned>(p.m) * p.n));
            const int bx = static_cast<int>(x.GetNumElements() / (x.GetShape()[rx - 1] * x.GetShape()[rx - 2]));
            const int by = static_cast<int>(y.GetNumElements() / (y.GetShape()[ry - 1] * y.GetShape()[ry - 2]));
            p.batch_stride_x = (bx == p.batch && p.batch > 1) ? static_cast<int64_t>(p.m) * p.k : 0;
            p.batch_stride_y = (by == p.batch && p.batch > 1) ? static_cast<int64_t>(p.k) * p.n : 0;
            const bool f32 = info.m_OutputTensorInfos[0].GetDataType() == DataType::Float32;
            return Make<BatchMatMulQueueDescriptor>(d, info, ctx, [st, f32](const BatchMatMulQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Inputs[1]); st->p.out.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(f32 ? b200k_batch_matmul_f32(&st->p, s) : b200k_batch_matmul_q8(&st->p, s));
            });
        }
        case LayerType::Pad:
        {
            // only Pad layers that B200Backend::OptimizeSubgraphView could not fold into their consumer get here
            const auto& qd = *PolymorphicDowncast<const PadQueueDescriptor*>(&d);
            auto st = std::make_shared<SimpleState<b200k_pad_params>>(ctx);
            b200k_pad_params& p = st->p;
            std::memset(&p, 0, sizeof(p));
            const TensorInfo& x = info.m_InputTensorInfos[0];
            p.x = Operand(x, st->blobs); p.y = Operand(info.m_OutputTensorInfos[0], st->blobs);
            p.rank = static_cast<int32_t>(x.GetNumDimensions());
            if (p.rank > 4 || qd.m_Parameters.m_PadList.size() != x.GetNumDimensions())
            {
                throw InvalidArgumentException("B200Acc: Pad needs rank <= 4 and one (before, after) pair per dimension");
            }
            for (int i = 0; i < p.rank; ++i)
            {
                p.shape[i] = x.GetShape()[i];
                p.pad_before[i] = qd.m_Parameters.m_PadList[i].first;
                p.pad_after[i] = qd.m_Parameters.m_PadList[i].second;
            }
            p.pad_value = qd.m_Parameters.m_PadValue;
            p.mode = qd.m_Parameters.m_PaddingMode == PaddingMode::Reflect ? 1 : qd.m_Parameters.m_PaddingMode == PaddingMode::Symmetric ? 2 : 0;
            return Make<PadQueueDescriptor>(d, info, ctx, [st](const PadQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_pad_q(&st->p, s));
            });
        }
        case LayerType::Resize:
        {
            const auto& qd = *PolymorphicDowncast<const ResizeQueueDescriptor*>(&d);
            auto st = std::make_shared<SimpleState<b200k_resize_params>>(ctx);
            b200k_resize_params& p = st->p;
            std::memset(&p, 0, sizeof(p));
            const TensorInfo& x = info.m_InputTensorInfos[0];
            const TensorInfo& y = info.m_OutputTensorInfos[0];
            p.x = Operand(x, st->blobs); p.y = Operand(y, st->blobs);
            const bool nchw = qd.m_Parameters.m_DataLayout == DataLayout::NCHW;
            const unsigned int hi = nchw ? 2 : 1, wi = nchw ? 3 : 2, ci = nchw ? 1 : 3;
            p.n = static_cast<int32_t>(x.GetShape()[0]); p.c = static_cast<int32_t>(x.GetShape()[ci]);
            p.in_h = static_cast<int32_t>(x.GetShape()[hi]); p.in_w = static_cast<int32_t>(x.GetShape()[wi]);
            p.out_h = static_cast<int32_t>(y.GetShape()[hi]); p.out_w = static_cast<int32_t>(y.GetShape()[wi]);
            p.method = qd.m_Parameters.m_Method == ResizeMethod::Bilinear ? 0 : 1;
            p.align_corners = qd.m_Parameters.m_AlignCorners ? 1 : 0;
            p.half_pixel_centers = qd.m_Parameters.m_HalfPixelCenters ? 1 : 0;
            p.nchw = nchw ? 1 : 0;
            return Make<ResizeQueueDescriptor>(d, info, ctx, [st](const ResizeQueueDescriptor& data, cudaStream_t s)
            {
                st->p.x.data = Dev(data.m_Inputs[0]); st->p.y.data = Dev(data.m_Outputs[0]);
                B200CheckStatus(b200k_resize_q(&st->p, s));
            });
        }
        case LayerType::Concat:       return MakeConcat(d, info, ctx);
        case LayerType::Splitter:     return MakeSplitter(d, info, ctx);
        case LayerType::Permute:      return MakePermute<PermuteQueueDescriptor>(d, info, ctx, false);
        case LayerType::Transpose:    return MakePermute<TransposeQueueDescriptor>(d, info, ctx, true);
        case LayerType::StridedSlice: return MakeStridedSlice(d, info, ctx);
        case LayerType::Slice:        return MakeSlice(d, info, ctx);
        case LayerType::DepthToSpace: return MakeDepthSpace<DepthToSpaceQueueDescriptor>(d, info, ctx, true);
        case LayerType::SpaceToDepth: return MakeDepthSpace<SpaceToDepthQueueDescriptor>(d, info, ctx, false);
        case LayerType::BatchToSpaceNd:
        {
            const auto& prm = PolymorphicDowncast<const BatchToSpaceNdQueueDescriptor*>(&d)->m_Parameters;
            return MakeBatchSpace<BatchToSpaceNdQueueDescriptor>(d, info, ctx, prm.m_BlockShape, prm.m_Crops, prm.m_DataLayout, true);
        }
        case LayerType::SpaceToBatchNd:
        {
            const auto& prm = PolymorphicDowncast<const SpaceToBatchNdQueueDescriptor*>(&d)->m_Parameters;
            return MakeBatchSpace<SpaceToBatchNdQueueDescriptor>(d, info, ctx, prm.m_BlockShape, prm.m_PadList, prm.m_DataLayout, false);
        }
        case LayerType::Tile:         return MakeTile(d, info, ctx);
        case LayerType::BroadcastTo:  return MakeBroadcastTo(d, info, ctx);
        case LayerType::ChannelShuffle: return MakeChannelShuffle(d, info, ctx);
        case LayerType::Stack:        return MakeStack(d, info, ctx);
        case LayerType::QLstm:
            return MakeQLstm(d, info, ctx);
        case LayerType::Lstm:
            return MakeLstm<LstmQueueDescriptor>(d, info, ctx, false);
        case LayerType::UnidirectionalSequenceLstm:
            return MakeLstm<UnidirectionalSequenceLstmQueueDescriptor>(d, info, ctx, true);
        case LayerType::PreCompiled:
        {
            const auto& qd = *PolymorphicDowncast<const PreCompiledQueueDescriptor*>(&d);
            const auto* fused = static_cast<const B200FusedConvAdd*>(qd.m_PreCompiledObject);
            if (!fused || fused->m_Magic != B200FusedConvAdd::Magic) { return nullptr; }
            return MakeFusedConvAdd(d, info, ctx, *fused);
        }
        default:
            return nullptr;       // LoadedNetwork turns a null workload into an exception: there is no CPU fallback
    }
}

}  // namespace armnn
