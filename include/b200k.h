/*
 * b200k.h — C ABI of libb200k.so, the sm_100a kernel library behind the Arm NN "B200Acc" backend.
 *
 * Every entry point is the device-side replacement of one CpuRef workload function of the
 * Arm NN reference (paths below are relative to the Arm NN source tree).  The B200Acc backend
 * plugin (armnn_b200/backend/, an IBackendInternal implementation) binds exactly these symbols:
 * one call per IWorkload::Execute().
 *
 * Conventions
 *  - plain C: raw device pointers, ints, floats; no C++ or torch types cross this line.
 *  - every launcher is asynchronous on the caller's CUDA stream (passed as void*, a cudaStream_t).
 *  - return value: 0 on success, a negative B200K_E_* code otherwise; never aborts, never throws.
 *    b200k_last_error() returns a thread-local description of the last failure.
 *  - tensors are dense, row-major, NHWC for 4-D image tensors (the only layout B200Acc accepts).
 *  - quantisation follows armnn::Quantize / armnn::Dequantize (src/armnn/TypesUtils.cpp:29-56):
 *        real = scale * (q - zero_point),   q = clamp(zero_point + round_half_away(real / scale)).
 *  - "clamp_lo/clamp_hi" carry a fused activation (ReLu / BoundedReLu) as a clamp in the output's
 *    quantised domain; use b200k_activation_clamp() to derive them.  Pass the type's full range
 *    for "no activation".
 */
#ifndef B200K_H
#define B200K_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200K_OK            0
#define B200K_E_INVALID    -1   /* bad argument (null pointer, unsupported dtype / shape) */
#define B200K_E_CUDA       -2   /* a CUDA runtime / driver call failed                      */
#define B200K_E_UNSUPPORTED -3  /* valid request that this library does not implement        */
#define B200K_E_NODEVICE   -4   /* no sm_100 device visible                                  */
#define B200K_E_TIMEOUT    -5   /* a bounded device-side wait gave up (status word set)      */
#define B200K_E_TOOBIG     -6   /* size beyond a documented fixed maximum                    */

/* element types; numbering is private to this ABI (armnn::DataType in include/armnn/Types.hpp) */
typedef enum {
    B200K_U8  = 0,  /* QAsymmU8                          */
    B200K_S8  = 1,  /* QAsymmS8 and QSymmS8              */
    B200K_S16 = 2,  /* QSymmS16                          */
    B200K_S32 = 3,  /* Signed32 (bias)                   */
    B200K_F32 = 4   /* Float32                           */
} b200k_dtype;

/* A quantised tensor operand.  `scales` (device pointer, one float per channel of the quantisation
 * axis) overrides `scale` when non-null: per-axis QSymmS8 weights and per-axis Signed32 bias
 * (src/backends/reference/workloads/BaseIterator.hpp:794-830, 861-911). */
typedef struct {
    const void*  data;        /* device pointer                              */
    int32_t      dtype;       /* b200k_dtype                                 */
    float        scale;       /* per-tensor scale                            */
    int32_t      zero_point;  /* per-tensor offset (0 for symmetric types)   */
    const float* scales;      /* device pointer, per-axis scales, or NULL    */
} b200k_qtensor;

/* ---- device management ------------------------------------------------------------------- */

/* Selects `device` for the calling thread and checks it is an sm_100 part.
 * Replaces nothing in CpuRef (RefBackend::CreateBackendContext returns null,
 * src/backends/reference/RefBackend.cpp:50-53); modelled on ClBackendContext
 * (src/backends/cl/ClBackendContext.cpp:61-215). */
int b200k_device_open(int device);
int b200k_device_count(void);
const char* b200k_last_error(void);
const char* b200k_version(void);

/* Quantised clamp range of a fused activation on an output tensor (scale, zero_point, dtype).
 * kind: 0 = none, 1 = ReLu, 2 = BoundedReLu(a = upper, b = lower)
 * (armnn::ActivationFunction, src/backends/reference/workloads/Activation.cpp:13-119).
 * Pure host arithmetic. */
int b200k_activation_clamp(int kind, float a, float b, float scale, int32_t zero_point,
                           int32_t dtype, int32_t* clamp_lo, int32_t* clamp_hi);

/* ---- Convolution2d / FullyConnected ------------------------------------------------------- */

/* armnn::Convolve, non-depthwise branch (src/backends/reference/workloads/ConvImpl.cpp:68-233),
 * called from RefConvolution2dWorkload::Execute (RefConvolution2dWorkload.cpp:33-58).
 *   x [n, h, w, c]  U8 or S8        w [oc, kh, kw, c]  U8 or S8, per-tensor or per-axis(dim 0)
 *   bias [oc] S32 with its own scale(s), or data == NULL       y [n, oh, ow, oc]  U8 or S8
 * acc = sum over in-bounds taps of (x - zx)(w - zw)   (int32, exact)
 * y   = clamp(zy + round((float(acc) * (sx * sw[oc]) + float(bias) * sb[oc]) / sy), lo, hi)
 * all in IEEE fp32 without fused multiply-add.
 * acc_out (optional, device int32 [n*oh*ow*oc]) receives the raw accumulators. */
typedef struct {
    b200k_qtensor x, w, bias, y;
    int32_t n, h, wd, c;            /* input  N H W C  */
    int32_t oh, ow, oc;             /* output H W C    */
    int32_t kh, kw;
    int32_t stride_h, stride_w;
    int32_t pad_top, pad_left;
    int32_t dil_h, dil_w;
    int32_t clamp_lo, clamp_hi;
    int32_t* acc_out;
    int32_t algo;                   /* 0 = auto, 1 = CUDA-core dp4a kernel, 2 = tcgen05 kernel */
    const void* packed;             /* optional result of b200k_conv2d_pack (device), or NULL   */
    /* Fused ElementwiseBinary Add (Convolution2d only; add_operand.data == NULL: none).  The convolution's own
     * 8-bit result q = Q_y(conv) is formed with y's scale / zero point but not stored (y.data is ignored), then
     *     add_out = clamp(Q_out(deq_y(q) + deq(add_operand)))
     * exactly as RefConvolution2dWorkload followed by RefElementwiseBinaryWorkload (and a ReLu / BoundedReLu
     * Activation expressed through clamp_lo / clamp_hi, which then refer to add_out) would produce.
     * add_operand and add_out have the convolution's output shape (no broadcast). */
    b200k_qtensor add_operand, add_out;
    /* Per-call device scratch (b200k_conv2d_scratch_bytes() bytes, 16-byte aligned; 0 for most layers): zero-padded
     * copies for channel counts that are multiples of 8 but not of 16, and the re-packed input of those few-channel
     * stems that the direct stem kernel cannot take (asymmetric per-tensor weights, a fused Add, rows that are not a
     * multiple of 16 bytes).  NULL or too small: such convolutions run on the CUDA-core kernel. */
    void* scratch;
    size_t scratch_bytes;
    /* Self-test of the bounded device-side waits of the tcgen05 kernel; 0 (the normal case) switches it off.  With
     * selftest_us > 0 the kernel's TMA producers issue no loads and every device-side wait gives up after about
     * selftest_us microseconds: the launch ends by itself, its output is meaningless, and the next
     * b200k_poll_status() returns B200K_E_TIMEOUT.  This is the failure a broken pipeline would produce, injected
     * from the host; nothing faults, traps or spins without a limit.  Ignored by the CUDA-core kernels. */
    int32_t selftest_us;
} b200k_conv2d_params;

int b200k_conv2d_q8(const b200k_conv2d_params* p, void* stream);

/* Load-time weight preparation for the tcgen05 path: per-tap per-channel weight sums as a 2-D
 * prefix table, int32 [(kh+1)*(kw+1)*oc], used to correct for zero-filled padding when zx != 0.
 * CpuRef re-decodes the weights on every inference (ConvImpl.cpp:111-115); this replaces that.
 * `packed` must hold b200k_conv2d_pack_bytes() bytes of device memory; only w, oc, kh, kw, c of the
 * parameter struct are read.  Without a packed table, convolutions whose input zero point is not 0
 * run on the CUDA-core kernel. */
size_t b200k_conv2d_pack_bytes(int32_t oc, int32_t kh, int32_t kw, int32_t c);
int b200k_conv2d_pack(const b200k_conv2d_params* p, void* packed, void* stream);
/* Bytes of per-call scratch b200k_conv2d_q8 wants for this geometry (0 for most shapes).  For c <= 16 the packed
 * table additionally holds the weights re-laid-out per filter row, which depends on kw, c and stride_w: those
 * must be set when calling b200k_conv2d_pack. */
size_t b200k_conv2d_scratch_bytes(const b200k_conv2d_params* p);

/* Same operation as b200k_conv2d_q8 for callers that cannot hand over freshly allocated device buffers (a memory
 * pool frozen before models are loaded, an allocator that is off limits after start-up).  p->packed and p->scratch
 * are ignored: the weight table is rebuilt on every call and, like the re-packed input, lives in a 16 MiB device
 * array built into the library (1 MiB for the table, 15 MiB for the input; every GPU that loads the library holds
 * it until the process exits).  Shapes needing more return B200K_E_TOOBIG.  No cudaMalloc / cudaFree happens
 * inside.  The first call on each device looks up the array's device address and should therefore come before any
 * stream capture.  All calls share the array: calls that may overlap on the GPU (different streams) race.
 * This entry point has no counterpart in the reference. */
int b200k_conv2d_q8_static(const b200k_conv2d_params* p, void* stream);

/* armnn::FullyConnected (src/backends/reference/workloads/FullyConnected.cpp:13-65) from
 * RefFullyConnectedWorkload::Execute (RefFullyConnectedWorkload.cpp:16-67).
 *   x [m, k]   w [n, k] when transpose_w != 0 (m_TransposeWeightMatrix) else [k, n]
 *   bias [n] or NULL   y [m, n];  per-axis weight scales index n.
 * Same arithmetic and epilogue as b200k_conv2d_q8.  With at most 16 rows (and [n, k] weights, k a multiple of 64) the
 * layer runs on a weight-streaming kernel instead of the convolution kernels when algo == 0. */
typedef struct {
    b200k_qtensor x, w, bias, y;
    int32_t m, k, n;
    int32_t transpose_w;
    int32_t clamp_lo, clamp_hi;
    int32_t* acc_out;
    int32_t algo;                   /* as b200k_conv2d_params.algo */
    const void* packed;             /* optional result of b200k_conv2d_pack for the [n, 1, 1, k] weights, or NULL */
} b200k_fc_params;

int b200k_fully_connected_q8(const b200k_fc_params* p, void* stream);

/* armnn::BatchMatMul (src/backends/reference/workloads/BatchMatMulImpl.cpp:15-139, 329-468) from
 * RefBatchMatMulWorkload::Execute (RefBatchMatMulWorkload.cpp:19-47).
 *   x [batch, m, k] (or [batch, k, m] when transpose_x), y [batch, k, n] (or [batch, n, k] when
 *   transpose_y), out [batch, m, n]; batch_stride_* = 0 broadcasts that operand.
 * Adjoint inputs are not implemented (the backend's layer-support predicate refuses them). */
typedef struct {
    b200k_qtensor x, y, out;
    int32_t batch, m, k, n;
    int32_t transpose_x, transpose_y;
    int64_t batch_stride_x, batch_stride_y;   /* elements; 0 = broadcast */
    int32_t* acc_out;
    int32_t algo;                             /* 0 = tensor-core kernel (mma.sync on 128 x 128 tiles, either layout of
                                                 either operand), 1 = the CUDA-core kernel */
} b200k_bmm_params;

int b200k_batch_matmul_q8(const b200k_bmm_params* p, void* stream);

/* The same on Float32 tensors: every output is the sum over k, in order, of separately rounded products
 * (BatchMatMulImpl.cpp:15-139); acc_out and algo are ignored. */
int b200k_batch_matmul_f32(const b200k_bmm_params* p, void* stream);

/* ---- DepthwiseConvolution2d ---------------------------------------------------------------- */

/* armnn::Convolve with depthwise = true (ConvImpl.cpp:100, 128-146) from
 * RefDepthwiseConvolution2dWorkload::Execute (RefDepthwiseConvolution2dWorkload.cpp:38-62).
 *   x [n, h, w, c]   w [1, kh, kw, oc], oc = c * depth_multiplier, per-axis scales index oc (dim 3)
 * Same epilogue as b200k_conv2d_q8. */
int b200k_dwconv2d_q8(const b200k_conv2d_params* p, void* stream);

/* ---- Pooling2d / Mean ----------------------------------------------------------------------- */

/* armnn::Pooling2d (src/backends/reference/workloads/Pooling2d.cpp:142-303).
 * pool_type: 0 Max, 1 Average, 2 L2 (armnn::PoolingAlgorithm)
 * padding_method: 0 IgnoreValue, 1 Exclude (armnn::PaddingMethod)
 * fp32 arithmetic in CpuRef's own summation order, so results equal CpuRef's bit for bit. */
typedef struct {
    b200k_qtensor x, y;
    int32_t n, h, wd, c, oh, ow;
    int32_t pool_h, pool_w, stride_h, stride_w;
    int32_t pad_top, pad_bottom, pad_left, pad_right;
    int32_t pool_type, padding_method;
} b200k_pool2d_params;

int b200k_pool2d_q8(const b200k_pool2d_params* p, void* stream);

/* armnn::Reduce with ReduceOperation::Mean over axes {1,2} of an NHWC tensor
 * (src/backends/reference/workloads/Reduce.cpp:68-173, RefMeanWorkload.cpp:22-38).
 * x [n, h, w, c] -> y [n, c] (keep_dims only changes the shape metadata). */
typedef struct {
    b200k_qtensor x, y;
    int32_t n, h, wd, c;
} b200k_mean_params;

int b200k_mean_hw_q8(const b200k_mean_params* p, void* stream);

/* ---- Convolution3d, Pooling3d --------------------------------------------------------------- */

/* armnn::Convolve3d (src/backends/reference/workloads/Conv3dImpl.cpp:14-177), DataLayout::NDHWC: x [n, d, h, wd, c],
 * weights [kd, kh, kw, c, oc] (per-tensor, or per-axis scales along oc), bias [oc] Signed32, y [n, od, oh, ow, oc].
 * Quantised tensors: exact int32 accumulation of (x - zx)(w - zw) and the epilogue of b200k_conv2d_q8; Float32
 * throughout: the reference's term order (z, y, x, input channel), products and sums rounded separately. */
typedef struct {
    b200k_qtensor x, w, bias, y;
    int32_t n, d, h, wd, c;
    int32_t od, oh, ow, oc;
    int32_t kd, kh, kw;
    int32_t stride_d, stride_h, stride_w;
    int32_t pad_front, pad_top, pad_left;
    int32_t dil_d, dil_h, dil_w;
    int32_t clamp_lo, clamp_hi;
} b200k_conv3d_params;

int b200k_conv3d_q(const b200k_conv3d_params* p, void* stream);

/* armnn::Pooling3d (src/backends/reference/workloads/Pooling3d.cpp:138-328), DataLayout::NDHWC.  pool_type and
 * padding_method as in b200k_pool2d_params; a window that lies in the padding only yields 0. */
typedef struct {
    b200k_qtensor x, y;
    int32_t n, d, h, wd, c;
    int32_t od, oh, ow;
    int32_t pool_d, pool_h, pool_w, stride_d, stride_h, stride_w;
    int32_t pad_front, pad_back, pad_top, pad_bottom, pad_left, pad_right;
    int32_t pool_type, padding_method;
} b200k_pool3d_params;

int b200k_pool3d_q(const b200k_pool3d_params* p, void* stream);

/* ---- ElementwiseBinary / Activation ------------------------------------------------------- */

/* ElementwiseBinaryFunction<std::plus / std::multiplies / ...> with BroadcastLoop
 * (RefElementwiseBinaryWorkload.cpp:27-132, ElementwiseFunction.cpp:25-34, Broadcast.hpp:13-104).
 * op follows armnn::BinaryOperation (include/armnn/Types.hpp:138-149): 0 Add, 1 Div, 2 Maximum,
 * 3 Minimum, 4 Mul, 5 Sub, 6 SqDiff, 7 Power (Power.hpp:19-24), 8 FloorDiv (FloorDiv.hpp:15-19: the quotient in
 * double precision, floored); B200K_ELTWISE_PRELU is armnn::Prelu (PreluImpl.cpp:14-33): a < 0 ? b * a : a with b the
 * alpha tensor; 200 + armnn::ComparisonOperation (0 Equal, 1 Greater, 2 GreaterOrEqual, 3 Less, 4 LessOrEqual,
 * 5 NotEqual; RefComparisonWorkload.cpp) and 210 + armnn::LogicalBinaryOperation (0 LogicalAnd, 1 LogicalOr;
 * RefLogicalBinaryWorkload.cpp) produce 1.0 or 0.0.  A Boolean tensor is a B200K_U8 tensor with scale 1 and zero point 0:
 * one byte per element, non-zero = true, results 0 or 1 (BooleanDecoder / BooleanEncoder, BaseIterator.hpp:427-700).
 * Shapes have equal rank <= 4 (padded with leading 1s); a dimension of size 1 broadcasts.
 * out = Q(deq(a) op deq(b)), then the clamp. */
#define B200K_ELTWISE_PRELU 100
typedef struct {
    b200k_qtensor a, b, out;
    int32_t rank;
    int32_t shape_a[4], shape_b[4], shape_out[4];
    int32_t op;
    int32_t clamp_lo, clamp_hi;
} b200k_eltwise_params;

int b200k_eltwise_q8(const b200k_eltwise_params* p, void* stream);

/* armnn::Activation (src/backends/reference/workloads/Activation.cpp:13-119).
 * function follows armnn::ActivationFunction numbering (include/armnn/Types.hpp):
 * 0 Sigmoid, 1 TanH, 2 Linear, 3 ReLu, 4 BoundedReLu, 5 SoftReLu, 6 LeakyReLu, 7 Abs, 8 Sqrt,
 * 9 Square, 10 Elu, 11 HardSwish, 12 Gelu (x / 2 * (1 + erf(x / sqrt(2))), the quotient in double precision).
 * B200K_ACTIVATION_FAKE_QUANTIZATION is the FakeQuantization layer (RefFakeQuantizationFloat32Workload.cpp:15-27), Float32
 * only: a = min, b = max; y = float(Quantize<uint8>(x, (max - min) / 255, int(-min * 255 / (max - min)))). */
#define B200K_ACTIVATION_FAKE_QUANTIZATION 50
typedef struct {
    b200k_qtensor x, y;
    int64_t count;
    int32_t function;
    float a, b;
} b200k_activation_params;

int b200k_activation_q8(const b200k_activation_params* p, void* stream);

/* armnn::ElementwiseUnary (src/backends/reference/workloads/RefElementwiseUnaryWorkload.cpp:36-110 with Abs.hpp, Exp.hpp,
 * Sqrt.hpp, Rsqrt.hpp, Log.hpp, Sin.hpp, Ceil.hpp and std::negate): y = Q_y(f(deq_x(x))); operation follows
 * armnn::UnaryOperation (0 Abs, 1 Exp, 2 Sqrt, 3 Rsqrt = 1 / sqrt, 4 Neg, 5 LogicalNot of a Boolean tensor
 * (B200K_U8, scale 1, zero point 0; RefLogicalUnaryWorkload.cpp), 6 Log, 7 Sin, 8 Ceil); 9 is the separate armnn::Floor layer (RefFloorWorkload.cpp: floorf). */
typedef struct {
    b200k_qtensor x, y;
    int64_t count;
    int32_t operation;
} b200k_unary_params;

int b200k_unary_q(const b200k_unary_params* p, void* stream);

/* armnn::Pad with PaddingMode::Constant (src/backends/reference/workloads/Pad.cpp:21-170, RefPadWorkload.cpp):
 * y has shape[d] + pad_before[d] + pad_after[d] elements along dimension d (rank <= 4, outermost first); elements
 * outside the copied block hold pad_value — for a quantised y a quantised number already (the reference encodes it with
 * scale 1 and offset 0, Pad.cpp:76-83; the TfLite parser passes the zero point) —, the others Q_y(deq_x(x)).
 * (Pad layers in front of a convolution or pooling layer never reach this: the backend folds them into the layer.) */
typedef struct {
    b200k_qtensor x, y;
    int32_t rank;
    int32_t shape[4];
    int32_t pad_before[4], pad_after[4];
    float pad_value;
    int32_t mode;               /* armnn::PaddingMode: 0 Constant, 1 Reflect, 2 Symmetric (MirrorPad.cpp:42-150; pad_value unused) */
} b200k_pad_params;

int b200k_pad_q(const b200k_pad_params* p, void* stream);

/* ---- Concat, Splitter, Permute, Transpose, StridedSlice, Slice, DepthToSpace, SpaceToDepth, ChannelShuffle, Stack,
 *      BatchToSpaceNd, SpaceToBatchNd ---- */

/* One rectangular view of a tensor copied onto a view of another one:
 *     y[dst_offset + sum_d i_d dst_strides[d]] = Q_y(deq_x(x[src_offset + sum_d i_d src_strides[d]]))   for 0 <= i_d < shape[d]
 * (offsets and strides in elements, outermost dimension first, rank <= 6; strides may be negative or zero).  With equal
 * quantisation the bytes are copied as they are.  This is what the reference's data-movement workloads do element by
 * element through a Decoder / Encoder pair or with memcpy:
 *   armnn::Concatenate (src/backends/reference/workloads/Concatenate.cpp:14-85): one call per input view, the
 *     destination view placed at the view's origin in the output;
 *   armnn::Split (workloads/Splitter.cpp:18-93): one call per output view, the source view at the origin in the input;
 *   armnnUtils::Permute / Transpose (src/armnnUtils/Permute.cpp:22-119, Transpose.cpp:22-117; RefPermuteWorkload.cpp,
 *     RefTransposeWorkload.cpp): the source strides in the destination's order of dimensions;
 *   armnn::StridedSlice (workloads/StridedSlice.cpp:90-223) and armnn::Slice (workloads/Slice.cpp:14-147): source
 *     offset from the begin indices, source strides multiplied by the slice's strides;
 *   armnn::DepthToSpace (workloads/DepthToSpace.cpp:15-100), SpaceToDepth (workloads/SpaceToDepth.cpp:42-104),
 *     ChannelShuffle (RefChannelShuffleWorkload.cpp:28-76): six- or four-dimensional walks over the same elements;
 *   armnn::Stack (workloads/Stack.cpp:14-120): one call per input, placed at its index of the new dimension;
 *   armnn::BatchToSpaceNd (workloads/BatchToSpaceNd.cpp:50-117) and SpaceToBatchNd (workloads/SpaceToBatchNd.cpp:49-131):
 *     one strided block per position inside the spatial block (a single six-dimensional walk without crops); the
 *     padding of SpaceToBatchNd is a fill from one element holding Q_y(0.0), read with source strides 0.
 * The host side (the plugin's workloads, armnn_b200/views.py) turns the layer descriptors into these views. */
typedef struct {
    b200k_qtensor x, y;
    int32_t rank;
    int32_t shape[6];
    int64_t src_strides[6], dst_strides[6];
    int64_t src_offset, dst_offset;
} b200k_view_copy_params;

int b200k_view_copy_q(const b200k_view_copy_params* p, void* stream);

/* ---- Float32 Convolution2d / DepthwiseConvolution2d / FullyConnected ------------------------- */

/* The fp32 variants of the contractions: every tensor Float32 (x, w, y and the optional bias), same parameter structs,
 * NHWC.  The sum runs in the reference's own order with a rounded product and a rounded sum per term
 * (sum += w * x over input channel, filter row, filter column: src/backends/reference/workloads/ConvImpl.cpp:118-204;
 * over the input channel: workloads/FullyConnected.cpp:32-58), so the results are CpuRef's bit for bit; padding taps
 * add w * 0.  CUDA-core kernels: correctness and coverage, not throughput.  clamp_lo / clamp_hi, add_operand, packed,
 * scratch and algo are unused (activations stay layers of their own for fp32 tensors). */
int b200k_conv2d_f32(const b200k_conv2d_params* p, void* stream);
int b200k_dwconv2d_f32(const b200k_conv2d_params* p, void* stream);
int b200k_fully_connected_f32(const b200k_fc_params* p, void* stream);

/* ---- TransposeConvolution2d ----------------------------------------------------------------- */

/* armnn::TransposeConvolution2dImpl (src/backends/reference/workloads/TransposeConvolution2d.cpp:14-160), NHWC,
 * weights [OC, KH, KW, C]: every input pixel (yi, xi) adds x * w to the outputs (yi * stride_h - pad_top + ky,
 * xi * stride_w - pad_left + kx) that lie inside the output; then the bias; then Q_y.  Takes the convolution's parameter
 * struct: h, wd are the input's and oh, ow the output's extents; dilation, add_operand, packed, scratch, algo are unused.  Like the
 * other contractions: exact int32 accumulation of (x - zx)(w - zw), one fp32 requantisation. */
int b200k_transpose_conv2d_q8(const b200k_conv2d_params* p, void* stream);

/* ---- Reduce ----------------------------------------------------------------------------------- */

/* armnn::Reduce (src/backends/reference/workloads/Reduce.cpp:63-175, RefReduceWorkload.cpp): op follows
 * armnn::ReduceOperation (0 Sum, 1 Max, 2 Mean, 3 Min, 4 Prod) over the dimensions whose bit is set in axis_mask (0: all
 * of them).  Every input element is decoded to fp32 and folded into its output's fp32 accumulator in the order of the
 * flat input index (the order matters for Sum, Mean and Prod); Mean divides by the number of folded elements; the
 * result is encoded with y's quantisation.  The output holds the kept dimensions in order (keep_dims only changes its
 * shape, not its bytes). */
typedef struct {
    b200k_qtensor x, y;
    int32_t rank;
    int32_t shape[6];
    int32_t axis_mask;
    int32_t op;
} b200k_reduce_params;

int b200k_reduce_q(const b200k_reduce_params* p, void* stream);

/* ---- Resize ----------------------------------------------------------------------------------- */

/* armnn::Resize (src/backends/reference/workloads/Resize.cpp:72-216): bilinear (method 0) or nearest-neighbour
 * (method 1, armnn::ResizeMethod) resampling of H and W, NHWC (nchw = 0) or NCHW; every sample is decoded to fp32,
 * interpolated with the reference's own sequence of fp32 operations (Lerp = w * b + (1 - w) * a, unfused) and encoded
 * with y's quantisation.  align_corners and half_pixel_centers as in armnn::ResizeDescriptor (not both). */
typedef struct {
    b200k_qtensor x, y;
    int32_t n, c, in_h, in_w, out_h, out_w;
    int32_t method;
    int32_t align_corners, half_pixel_centers;
    int32_t nchw;
} b200k_resize_params;

int b200k_resize_q(const b200k_resize_params* p, void* stream);

/* armnn::ScatterNd (src/backends/reference/workloads/ScatterNd.cpp:37-333), without the axis option (which the reference
 * refuses too).  y [dims[0] .. dims[nd-1], inner] starts as x (x.data == NULL: as zeros, the variant whose first input is
 * a shape), then tuple j of indices [n_indices, nd] replaces its slice:
 *     y[tuple j, k] = Q_y(function(base[tuple j, k], deq(updates[j, k]))),  base = deq_x(x) or 0
 * function follows armnn::ScatterNdFunction: 0 Update, 1 Add, 2 Sub, 3 Max, 4 Min, 5 Mul.  The base is the input, not the
 * running output, so of several tuples that address one slice the last one decides (for Update the reference throws on
 * such duplicates; a tuple outside the tensor, on which it throws as well, is skipped here). */
typedef struct {
    b200k_qtensor x, updates, y;
    const int32_t* indices;
    int32_t n_indices, nd, inner;
    int32_t dims[8];
    int32_t function;
} b200k_scatter_nd_params;

int b200k_scatter_nd_q(const b200k_scatter_nd_params* p, void* stream);

/* armnn::ReverseV2 (src/backends/reference/workloads/ReverseV2Impl.cpp:14-133): y is x mirrored along every dimension
 * listed in `axes` (device int32, n_axes entries, negative ones counted from the end; the layer's second input). */
typedef struct {
    b200k_qtensor x, y;
    const int32_t* axes;
    int32_t n_axes, rank;
    int32_t shape[6];
} b200k_reverse_params;

int b200k_reverse_q(const b200k_reverse_params* p, void* stream);

/* armnn::Gather (src/backends/reference/workloads/Gather.cpp:16-94): with x seen as [outer, axis_size, inner],
 *     y[o, j, k] = Q_y(deq_x(x[o, indices[j], k]))        0 <= j < n_indices
 * indices: device int32 (Signed32 tensor), a negative one counts from the end of the axis.  The reference throws on an
 * index outside the axis (its workload, RefGatherWorkload.cpp:40-47, on any negative index); here that position of y holds the
 * encoding of 0.0 and nothing is read. */
typedef struct {
    b200k_qtensor x, y;
    const int32_t* indices;
    int32_t outer, axis_size, inner, n_indices;
} b200k_gather_params;

int b200k_gather_q(const b200k_gather_params* p, void* stream);

/* armnn::GatherNd without batch dimensions (src/backends/reference/workloads/RefGatherNdWorkload.cpp:20-92): indices is
 * [n_indices, nd] (device int32); tuple j addresses the first nd dimensions (extents dims[0 .. nd-1]) of x, and
 *     y[j, k] = Q_y(deq_x(x[tuple j flattened, k]))        0 <= k < inner = product of the remaining dimensions.
 * A tuple outside the tensor (the reference throws on a negative entry) yields the encoding of 0.0. */
typedef struct {
    b200k_qtensor x, y;
    const int32_t* indices;
    int32_t n_indices, nd, inner;
    int32_t dims[8];
} b200k_gather_nd_params;

int b200k_gather_nd_q(const b200k_gather_nd_params* p, void* stream);

/* ---- BatchNormalization, InstanceNormalization ------------------------------------------------ */

/* armnn::BatchNormImpl (src/backends/reference/workloads/BatchNormImpl.cpp:16-63): per channel
 *     mult = gamma / sqrt(variance + eps), add = beta - mult * mean, y = Q_y(mult * deq_x(x) + add)
 * on a tensor [n, hw, c] (nchw = 0) or [n, c, hw] (nchw = 1); mean, variance, beta, gamma: [c] tensors of any supported
 * type.  scratch: 2 * c floats of device memory the call may overwrite (the per-channel constants). */
typedef struct {
    b200k_qtensor x, y, mean, variance, beta, gamma;
    int32_t n, c;
    int64_t hw;
    int32_t nchw;
    float eps;
    void* scratch;
} b200k_batch_norm_params;

int b200k_batch_norm_q(const b200k_batch_norm_params* p, void* stream);

/* armnn::InstanceNorm (src/backends/reference/workloads/InstanceNorm.cpp:16-84): per (batch, channel) plane the mean and
 * the (biased) variance over hw, summed in row-major order, then y = (x - mean) * gamma / sqrt(var + eps) + beta.
 * Float32 tensors only, as in the reference (InstanceNormalizationQueueDescriptor::Validate). */
typedef struct {
    b200k_qtensor x, y;
    int32_t n, c;
    int64_t hw;
    int32_t nchw;
    float gamma, beta, eps;
} b200k_instance_norm_params;

int b200k_instance_norm_q(const b200k_instance_norm_params* p, void* stream);

/* armnn::Normalization, LocalBrightness (src/backends/reference/workloads/RefNormalizationWorkload.cpp:19-140), with
 * r = norm_size / 2 and positions outside the tensor skipped:
 *   channel_type 0 (Across): s = sum of x^2 over channels c - r .. c + r of the pixel, y = x * powf(kappa + s * alpha, -beta);
 *   channel_type 1 (Within): s = sum of x^2 over the (2 r + 1)^2 window in the same channel, y = x / powf(kappa + s * alpha, beta);
 *     the reference indexes the tensor as NCHW whatever the descriptor's layout: pass c, h, w = shape[1], shape[2], shape[3]
 *     and nchw = 1.
 * The reference encodes the output with the INPUT's quantisation (line 176): a caller that wants its bytes passes x's
 * scale and zero point in y. */
typedef struct {
    b200k_qtensor x, y;
    int32_t n, c, h, w;
    int32_t nchw;
    int32_t channel_type;
    uint32_t norm_size;
    float alpha, beta, kappa;
} b200k_normalization_params;

int b200k_normalization_q(const b200k_normalization_params* p, void* stream);

/* ---- Softmax --------------------------------------------------------------------------------- */

/* armnn::Softmax (src/backends/reference/workloads/Softmax.cpp:17-70): softmax over the axis of
 * length `axis_size`, for outer x inner independent rows, element stride `inner` along the axis. */
typedef struct {
    b200k_qtensor x, y;
    int32_t outer, axis_size, inner;
    float beta;
} b200k_softmax_params;

int b200k_softmax_q8(const b200k_softmax_params* p, void* stream);

/* armnn::LogSoftmax (src/backends/reference/workloads/LogSoftmax.cpp:30-88): (x - max) * beta - log(sum exp((x - max) * beta))
 * over the same rows. */
int b200k_log_softmax_q(const b200k_softmax_params* p, void* stream);

/* armnn::L2Normalization (src/backends/reference/workloads/RefL2NormalizationWorkload.cpp:29-93): every element divided by
 * sqrt(max(sum of squares over the channel axis, eps)); the channel axis is the row axis here (NHWC: inner = 1, NCHW:
 * inner = H * W) and `beta` carries eps. */
int b200k_l2_normalization_q(const b200k_softmax_params* p, void* stream);

/* armnn::ArgMinMax (src/backends/reference/workloads/ArgMinMax.cpp:16-48): the index of the smallest (function 0) or
 * largest (function 1) decoded element of each row, the first one among equals; y is a device array of outer * inner
 * int32 (out_int64 = 0) or int64 (out_int64 = 1) indices. */
typedef struct {
    b200k_qtensor x;
    void* y;
    int32_t outer, axis_size, inner;
    int32_t function;
    int32_t out_int64;
} b200k_arg_min_max_params;

int b200k_arg_min_max_q(const b200k_arg_min_max_params* p, void* stream);

/* ---- Quantize / Dequantize ----------------------------------------------------------------- */

/* QuantizeImpl (RefQuantizeWorkload.cpp:14-45) and armnn::Dequantize
 * (src/backends/reference/workloads/Dequantize.cpp:11-28): any of F32/U8/S8/S16 -> any of
 * F32/U8/S8/S16 through fp32, i.e. quantize, dequantize and requantize in one entry point. */
typedef struct {
    b200k_qtensor x, y;
    int64_t count;
} b200k_convert_params;

int b200k_convert_q(const b200k_convert_params* p, void* stream);

/* armnn::ConvertFp16ToFp32 (to_half = 0: x holds IEEE binary16, y Float32; exact) and ConvertFp32ToFp16 (to_half = 1:
 * round to nearest, ties to even, and +-infinity — overflow or an infinite input — replaced by +-65504), as
 * armnnUtils::FloatingPointConverter does them
 * (src/armnnUtils/FloatingPointConverter.cpp:17-45, src/armnnUtils/Half.hpp:11-16).  With these two layers on the backend
 * the optimizer can run a Float16 network's layers in Float32 here instead of falling back. */
typedef struct {
    const void* x;
    void* y;
    int64_t count;
    int32_t to_half;
} b200k_convert_fp16_params;

int b200k_convert_fp16(const b200k_convert_fp16_params* p, void* stream);

/* armnn::Cast (src/backends/reference/workloads/RefCastWorkload.cpp:13-36, 95-106): the numbers stored in x become the
 * numbers stored in y: both tensors are read with scale 1 and offset 0 whatever x.scale / y.scale say, the value is
 * floored before an integer output (and clamped to the type's range), kept as it is for a float output.  Any of
 * U8/S8/S16/S32/F32 on either side. */
int b200k_cast_q(const b200k_convert_params* p, void* stream);

/* ---- QLstm ----------------------------------------------------------------------------------- */

/* One RefQLstmWorkload::Execute step (src/backends/reference/workloads/RefQLstmWorkload.cpp:46-541,
 * LstmUtils.cpp:16-256) reproduced operation by operation, including the re-quantisation of the
 * int16 gate buffers after every multiply-accumulate (LstmUtils.cpp:87-111).
 * Weight pointers are device pointers; a NULL pointer disables the corresponding option exactly as
 * the reference's m_CifgEnabled / m_PeepholeEnabled / m_ProjectionEnabled / m_LayerNormEnabled do. */
typedef struct {
    int32_t batch, input_size, num_units, output_size;
    /* tensors */
    /* gate bias scales s_b*: the reference derives them as layer-norm weight scale / 1024
     * (RefQLstmWorkload.cpp:261-287) and ignores the biases entirely without layer norm. */
    const int8_t*  input;            float input_scale;  int32_t input_zp;       /* [batch, input_size]  */
    const int8_t*  output_state_in;  float output_state_scale; int32_t output_state_zp; /* [batch, output_size] */
    const int16_t* cell_state_in;    float cell_state_scale;   /* [batch, num_units]  */
    int8_t*  output_state_out;       /* [batch, output_size], same quantisation as output_state_in */
    int16_t* cell_state_out;         /* [batch, num_units]   */
    int8_t*  output;                 float output_scale; int32_t output_zp;      /* [batch, output_size] */
    /* weights: int8 [num_units, input_size] / [num_units, output_size]; each with its scale */
    const int8_t *w_i2i, *w_i2f, *w_i2c, *w_i2o;   float s_i2i, s_i2f, s_i2c, s_i2o;
    const int8_t *w_r2i, *w_r2f, *w_r2c, *w_r2o;   float s_r2i, s_r2f, s_r2c, s_r2o;
    const int16_t *w_c2i, *w_c2f, *w_c2o;          float s_c2i, s_c2f, s_c2o;   /* peephole [num_units] */
    const int32_t *b_i, *b_f, *b_c, *b_o;          float s_bi, s_bf, s_bc, s_bo; /* gate biases          */
    const int16_t *ln_i, *ln_f, *ln_c, *ln_o;      float s_lni, s_lnf, s_lnc, s_lno; /* layer-norm w   */
    const int8_t  *w_proj;  float s_proj;          /* [output_size, num_units] */
    const int32_t *b_proj;  float s_bproj;
    /* descriptor (armnn::QLstmDescriptor, include/armnn/Descriptors.hpp) */
    float cell_clip, projection_clip;
    float input_intermediate_scale, forget_intermediate_scale, cell_intermediate_scale,
          output_intermediate_scale;
    float hidden_state_scale; int32_t hidden_state_zp;
} b200k_qlstm_params;

int b200k_qlstm_step(const b200k_qlstm_params* p, void* stream);

/* One step of armnn::LstmImpl on Float32 tensors (src/backends/reference/workloads/Lstm.cpp:14-259 with LstmUtils.cpp;
 * the Lstm layer, and every time step of UnidirectionalSequenceLstm): gate pre-activations accumulated term by term in
 * the reference's order (bias, input weights over the input, recurrent weights over the previous output, peephole),
 * optional layer normalisation, sigmoid gates, the cell activation, cell update and clipping, optional projection with
 * clipping.  Row-major matrices [rows = units (or outputs), columns].
 *   w_i2i == NULL: CIFG (no input gate; it becomes 1 - forget gate);  w_c2f == NULL: no peephole;
 *   ln_f == NULL: no layer normalisation;  w_proj == NULL: no projection (output_size == num_units then).
 *   activation (armnn::LstmDescriptor::m_ActivationFunc): 0 none, 1 ReLu, 3 ReLu6, 4 TanH, 6 Sigmoid.
 *   input_stride / output_stride: elements between the rows of two batch entries (a time step of a sequence tensor).
 * output_state_out / cell_state_out may be the state inputs themselves (the steps of a sequence update them in place).
 * The layer's scratch-buffer output is working memory in the reference and is not written. */
typedef struct {
    int32_t batch, input_size, num_units, output_size;
    const float* input; int64_t input_stride;
    const float* output_state_in; const float* cell_state_in;
    float* output_state_out; float* cell_state_out;
    float* output; int64_t output_stride;
    const float *w_i2i, *w_i2f, *w_i2c, *w_i2o;
    const float *w_r2i, *w_r2f, *w_r2c, *w_r2o;
    const float *w_c2i, *w_c2f, *w_c2o;
    const float *b_i, *b_f, *b_c, *b_o;
    const float *ln_i, *ln_f, *ln_c, *ln_o;
    const float *w_proj, *b_proj;
    int32_t activation;
    float cell_clip, projection_clip, layer_norm_eps;
} b200k_lstm_params;

int b200k_lstm_step_f32(const b200k_lstm_params* p, void* stream);

/* Status of the bounded device-side waits of the tcgen05 kernels: B200K_OK, or B200K_E_TIMEOUT when a wait
 * gave up since the last poll (the status word is then cleared).  Synchronises the device.  No counterpart in
 * the reference. */
int b200k_poll_status(void);

/* Measures what the tcgen05 int8 pipe of the current device sustains with nothing else in the way: one CTA per SM
 * issuing kind::i8 MMAs (128 x 256 x 32) back to back on resident shared-memory tiles for about a millisecond, best of
 * three repetitions, in TOP/s (2 x MAC).  The denominator of "fraction of the int8 tensor peak" figures.  Allocates a
 * status word and synchronises.  No counterpart in the reference. */
int b200k_int8_mma_peak(double* tops, void* stream);

/* Kernels this library has launched in this process so far (every launch of every entry point counts; a launch
 * recorded into a CUDA graph during stream capture counts once).  For callers that report how many of the library's
 * kernels a measured region ran.  No counterpart in the reference. */
unsigned long long b200k_kernel_launches(void);

/* sizeof() of a parameter struct as compiled into the library, for bindings in other languages to check their
 * own declarations: 0 conv2d, 1 fc, 2 bmm, 3 pool2d, 4 mean, 5 eltwise, 6 activation, 7 softmax, 8 convert,
 * 9 qlstm, 10 pad, 11 view_copy, 12 resize, 13 reduce, 14 unary, 15 arg_min_max, 16 gather, 17 batch_norm, 18 instance_norm, 19 normalization, 20 conv3d, 21 pool3d, 22 gather_nd, 23 lstm, 24 reverse, 25 convert_fp16, 26 scatter_nd.  No counterpart in the reference (its backends are linked as C++). */
size_t b200k_sizeof_params(int which);

#ifdef __cplusplus
}
#endif
#endif /* B200K_H */
