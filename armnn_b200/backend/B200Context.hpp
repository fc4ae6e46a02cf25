// Per-network execution context of the B200Acc backend: which GPU a LoadedNetwork runs on, the CUDA stream all of its
// workloads and transfers are enqueued on, and the replay of its workload queue as one CUDA graph.
//
// One context is created per LoadedNetwork, by B200Backend::CreateWorkloadFactory(registry, modelOptions, ...)
// (src/armnn/LoadedNetwork.cpp:264-279 of the Arm NN tree passes the network's ModelOptions there), and shared by that
// network's tensor-handle factory, tensor handles and workloads.  The device comes from the ModelOption
// BackendOptions("B200Acc", {{"DeviceId", n}}), else from the runtime-level BackendOption of the same name, else
// from the environment variable B200ACC_DEVICE_ID, else 0.  Several networks on several GPUs can live in one
// process, one host thread each (IRuntime::EnqueueWorkload locks per network, Runtime.cpp:580-586).
//
// Graph replay.  LoadedNetwork::Execute calls IWorkload::Execute() layer by layer; each B200 workload is one kernel
// launch (plus the host work around it).  After two ordinary inferences the context records the launches of the
// third one into a CUDA graph (stream capture), and from then on the first workload of an inference launches the
// whole graph while the others return at once: the per-layer host cost (parameter checks, tensor-map encoding, one
// driver call per kernel) is paid once instead of per inference.  The graph is dropped and recorded again when a
// tensor handle is replaced or imports another buffer; it is never used when a handle is mapped in the middle of the
// queue (a layer of another backend between two B200 layers) or while the Arm NN profiler is enabled.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <functional>
#include <memory>
#include <vector>

namespace armnn
{

class B200TensorHandle;

class B200Context
{
public:
    /// Throws BackendUnavailableException when the device is absent or not an sm_100 part.
    explicit B200Context(int deviceId);
    ~B200Context();
    B200Context(const B200Context&) = delete;
    B200Context& operator=(const B200Context&) = delete;

    int Device() const { return m_Device; }
    cudaStream_t Stream() const { return m_Stream; }
    void MakeCurrent() const;

    /// Counts inferences: an imported input is uploaded once per epoch.
    uint64_t Epoch() const { return m_Epoch; }

    // ---- the workload queue --------------------------------------------------------------------------
    /// A workload takes a position in its network's queue when it is created (creation order = execution order).
    /// `launches` says whether it enqueues GPU work at every inference (Constant workloads do not).
    int Register(bool launches);
    /// Runs workload `index`: `launch` enqueues its kernels on the given stream.  `reads` are the input handles of the
    /// workload (imported network inputs among them are brought to the device before the first launch).
    void Run(int index, const std::vector<const B200TensorHandle*>& reads, const std::function<void(cudaStream_t)>& launch);

    /// A handle of this network is being mapped: everything enqueued so far must have run.  Returns after the stream
    /// has been synchronised.  A map between the first and the last workload of an inference switches graph replay off.
    void SyncForMap();
    /// Device pointers behind the recorded graph changed (handle replaced, another buffer imported, memory re-acquired).
    void Invalidate();
    /// End of IRuntime::EnqueueWorkload (IBackendContext::AfterEnqueueWorkload): synchronise, report device-side errors,
    /// begin the next epoch.  Returns false after a device-side failure (bounded wait gave up, CUDA error).
    bool EndInference();

    /// Self-test option (runtime BackendOption "WaitSelfTestUs"): passed to every convolution as
    /// b200k_conv2d_params.selftest_us; 0 in normal operation.
    int SelfTestUs() const { return m_SelfTestUs; }

    bool GraphActive() const { return m_State == State::Replay; }
    uint64_t GraphLaunches() const { return m_GraphLaunches; }

    // ---- process-wide defaults and the list of live contexts -------------------------------------------
    static void SetDefaultDevice(int deviceId);         ///< runtime-level "DeviceId" (IBackendContext)
    static int DefaultDevice();
    static void SetDefaultSelfTestUs(int us);
    static void SetGraphReplayEnabled(bool on);         ///< runtime-level "GraphReplay" (default on)
    static bool EndInferenceAll();                      ///< every live context (AfterEnqueueWorkload has no network handle)
    static void SynchronizeAll();
    /// The context handles and workloads created through the legacy (non-registry) factory entry points share.
    static std::shared_ptr<B200Context> Shared();
    /// Process-wide counters for callers that report what ran: graph launches so far, and the kernel nodes they contained.
    static void Stats(uint64_t& graphLaunches, uint64_t& graphKernels);

private:
    enum class State { Warmup, Capture, Replay, Eager };

    void FinishCapture(bool launchIt);

    int m_Device = 0;
    cudaStream_t m_Stream = nullptr;
    uint64_t m_Epoch = 1;
    int m_SelfTestUs = 0;

    int m_Registered = 0;
    int m_First = -1, m_Last = -1;                       // first / last workload that launches GPU work
    State m_State = State::Warmup;
    int m_WarmInferences = 0;
    bool m_InFlight = false;                             // between the first and the last workload of an inference
    bool m_MappedInFlight = false;                       // a handle was mapped while in flight (this inference)
    bool m_Replaying = false;                            // this inference runs as a graph launch
    bool m_GraphAllowed = true;
    cudaGraphExec_t m_GraphExec = nullptr;
    std::vector<const B200TensorHandle*> m_ImportedInputs;   // uploaded before the graph is launched
    uint64_t m_GraphLaunches = 0;
    uint64_t m_GraphKernelNodes = 0;                     // kernel nodes of the recorded graph
};

}  // namespace armnn
