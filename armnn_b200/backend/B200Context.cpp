#include "B200Context.hpp"
#include "B200TensorHandle.hpp"

#include <armnn/Exceptions.hpp>
#include <Profiling.hpp>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <string>
#include <thread>

#include "b200k.h"

namespace armnn
{

namespace
{
std::atomic<int> g_DefaultDevice{-1};
std::atomic<int> g_DefaultSelfTestUs{0};
std::atomic<bool> g_GraphReplay{true};
std::atomic<uint64_t> g_TotalGraphLaunches{0}, g_TotalGraphKernels{0};
std::mutex g_ContextsMutex;
std::vector<B200Context*> g_Contexts;                    // live contexts (raw: a context removes itself)
std::weak_ptr<B200Context> g_Shared;

thread_local std::vector<B200Context*> t_Touched;       // contexts this thread has run workloads on since its last EndInferenceAll

bool ProfilerEnabled()
{
    IProfiler* p = ProfilerManager::GetInstance().GetProfiler();
    return p != nullptr && p->IsProfilingEnabled();
}
}  // namespace

void B200Context::SetDefaultDevice(int deviceId) { g_DefaultDevice.store(deviceId); }

int B200Context::DefaultDevice()
{
    int dev = g_DefaultDevice.load();
    if (dev < 0)
    {
        const char* env = std::getenv("B200ACC_DEVICE_ID");
        dev = env ? std::atoi(env) : 0;
    }
    return dev;
}

void B200Context::Stats(uint64_t& graphLaunches, uint64_t& graphKernels)
{
    graphLaunches = g_TotalGraphLaunches.load();
    graphKernels = g_TotalGraphKernels.load();
}

void B200Context::SetDefaultSelfTestUs(int us) { g_DefaultSelfTestUs.store(us); }
void B200Context::SetGraphReplayEnabled(bool on) { g_GraphReplay.store(on); }

std::shared_ptr<B200Context> B200Context::Shared()
{
    std::lock_guard<std::mutex> lock(g_ContextsMutex);
    std::shared_ptr<B200Context> ctx = g_Shared.lock();
    if (!ctx)
    {
        ctx = std::make_shared<B200Context>(DefaultDevice());
        g_Shared = ctx;
    }
    return ctx;
}

B200Context::B200Context(int deviceId)
{
    if (b200k_device_open(deviceId) != B200K_OK)
    {
        throw BackendUnavailableException(std::string("B200Acc: ") + b200k_last_error());
    }
    m_Device = deviceId;
    if (cudaStreamCreateWithFlags(&m_Stream, cudaStreamNonBlocking) != cudaSuccess)
    {
        throw BackendUnavailableException("B200Acc: cannot create a CUDA stream");
    }
    m_SelfTestUs = g_DefaultSelfTestUs.load();
    m_GraphAllowed = g_GraphReplay.load() && m_SelfTestUs == 0;
    std::lock_guard<std::mutex> lock(g_ContextsMutex);
    g_Contexts.push_back(this);
}

B200Context::~B200Context()
{
    {
        std::lock_guard<std::mutex> lock(g_ContextsMutex);
        g_Contexts.erase(std::remove(g_Contexts.begin(), g_Contexts.end(), this), g_Contexts.end());
    }
    t_Touched.erase(std::remove(t_Touched.begin(), t_Touched.end(), this), t_Touched.end());
    cudaSetDevice(m_Device);
    if (m_State == State::Capture) { FinishCapture(false); }
    if (m_Stream) { cudaStreamSynchronize(m_Stream); }
    if (m_GraphExec) { cudaGraphExecDestroy(m_GraphExec); }
    if (m_Stream) { cudaStreamDestroy(m_Stream); }
}

void B200Context::MakeCurrent() const
{
    B200Check(cudaSetDevice(m_Device), "cudaSetDevice");
}

int B200Context::Register(bool launches)
{
    const int index = m_Registered++;
    if (launches)
    {
        if (m_First < 0) { m_First = index; }
        m_Last = index;
    }
    return index;
}

void B200Context::FinishCapture(bool launchIt)
{
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(m_Stream, &graph);
    m_State = State::Eager;
    if (e != cudaSuccess || !graph)
    {
        cudaGetLastError();
        throw RuntimeException(std::string("B200Acc: recording the workload queue failed: ") + cudaGetErrorString(e));
    }
    size_t nodes = 0;
    m_GraphKernelNodes = 0;
    if (cudaGraphGetNodes(graph, nullptr, &nodes) == cudaSuccess && nodes > 0)
    {
        std::vector<cudaGraphNode_t> list(nodes);
        if (cudaGraphGetNodes(graph, list.data(), &nodes) == cudaSuccess)
        {
            for (size_t i = 0; i < nodes; ++i)
            {
                cudaGraphNodeType type;
                if (cudaGraphNodeGetType(list[i], &type) == cudaSuccess && type == cudaGraphNodeTypeKernel) { ++m_GraphKernelNodes; }
            }
        }
    }
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    B200Check(e, "cudaGraphInstantiate");
    if (launchIt)
    {
        // what was recorded has not run yet: run it now
        e = cudaGraphLaunch(exec, m_Stream);
        if (e != cudaSuccess) { cudaGraphExecDestroy(exec); B200Check(e, "cudaGraphLaunch"); }
    }
    if (m_GraphExec) { cudaGraphExecDestroy(m_GraphExec); }
    m_GraphExec = exec;
}

void B200Context::Run(int index, const std::vector<const B200TensorHandle*>& reads, const std::function<void(cudaStream_t)>& launch)
{
    MakeCurrent();
    if (index < m_First || index > m_Last || m_First < 0)
    {
        launch(m_Stream);                                // load-time work (Constant): not part of the recorded queue
        return;
    }
    if (std::find(t_Touched.begin(), t_Touched.end(), this) == t_Touched.end()) { t_Touched.push_back(this); }

    if (index == m_First)
    {
        m_InFlight = true;
        m_MappedInFlight = false;
        const bool profiling = ProfilerEnabled();
        if (m_State == State::Replay && !profiling)
        {
            for (const B200TensorHandle* h : m_ImportedInputs) { h->SyncImportedToDevice(); }
            B200Check(cudaGraphLaunch(m_GraphExec, m_Stream), "cudaGraphLaunch");
            ++m_GraphLaunches;
            g_TotalGraphLaunches.fetch_add(1, std::memory_order_relaxed);
            g_TotalGraphKernels.fetch_add(m_GraphKernelNodes, std::memory_order_relaxed);
            m_Replaying = true;
        }
        else
        {
            m_Replaying = false;
            if (m_State == State::Warmup && m_GraphAllowed && !profiling && m_WarmInferences >= 2)
            {
                // record this inference: network inputs that live in user memory are uploaded outside the graph
                for (const B200TensorHandle* h : m_ImportedInputs) { h->SyncImportedToDevice(); }
                B200Check(cudaStreamBeginCapture(m_Stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
                m_State = State::Capture;
            }
        }
    }

    if (!m_Replaying)
    {
        for (const B200TensorHandle* h : reads)
        {
            if (!h->IsImported()) { continue; }
            if (std::find(m_ImportedInputs.begin(), m_ImportedInputs.end(), h) == m_ImportedInputs.end())
            {
                if (m_State == State::Capture)
                {
                    // an imported input the warm-up passes have not seen: its upload must stay outside the graph
                    FinishCapture(true);
                    m_State = State::Warmup;
                    m_WarmInferences = 1;
                }
                m_ImportedInputs.push_back(h);
            }
            h->SyncImportedToDevice();
        }
        try
        {
            launch(m_Stream);
        }
        catch (...)
        {
            if (m_State == State::Capture)
            {
                // leave the stream usable: drop what has been recorded
                cudaGraph_t graph = nullptr;
                cudaStreamEndCapture(m_Stream, &graph);
                if (graph) { cudaGraphDestroy(graph); }
                cudaGetLastError();
                m_State = State::Eager;
                m_GraphAllowed = false;
            }
            m_InFlight = false;
            throw;
        }
    }

    if (index == m_Last)
    {
        if (m_State == State::Capture)
        {
            FinishCapture(true);
            m_State = State::Replay;
        }
        else if (m_State == State::Warmup && !m_MappedInFlight)
        {
            ++m_WarmInferences;
        }
        if (m_MappedInFlight && m_State != State::Replay)
        {
            // another backend's layer sits between two B200 layers: the queue cannot run ahead of the host
            m_GraphAllowed = false;
            m_State = State::Eager;
        }
        m_InFlight = false;
    }
}

void B200Context::SyncForMap()
{
    MakeCurrent();
    if (m_State == State::Capture)
    {
        FinishCapture(true);                             // run what has been recorded, then carry on without a graph
        m_GraphAllowed = false;
    }
    if (m_InFlight) { m_MappedInFlight = true; }
    B200Check(cudaStreamSynchronize(m_Stream), "cudaStreamSynchronize");
}

void B200Context::Invalidate()
{
    if (m_State == State::Capture) { return; }           // ends by itself; the next change invalidates again
    if (m_GraphExec)
    {
        cudaStreamSynchronize(m_Stream);
        cudaGraphExecDestroy(m_GraphExec);
        m_GraphExec = nullptr;
    }
    m_ImportedInputs.clear();
    if (m_State == State::Replay || m_State == State::Warmup)
    {
        m_State = State::Warmup;
        m_WarmInferences = std::min(m_WarmInferences, 1);
    }
}

bool B200Context::EndInference()
{
    cudaSetDevice(m_Device);
    if (m_State == State::Capture) { return true; }      // (not reached in practice: the last workload ends the capture)
    const bool ok = cudaStreamSynchronize(m_Stream) == cudaSuccess && b200k_poll_status() == B200K_OK;
    ++m_Epoch;
    m_InFlight = false;
    return ok;
}

bool B200Context::EndInferenceAll()
{
    bool ok = true;
    std::vector<B200Context*> mine;
    mine.swap(t_Touched);
    for (B200Context* c : mine)
    {
        {
            // a context may have gone with its network since this thread used it
            std::lock_guard<std::mutex> lock(g_ContextsMutex);
            if (std::find(g_Contexts.begin(), g_Contexts.end(), c) == g_Contexts.end()) { continue; }
        }
        ok = c->EndInference() && ok;
    }
    return ok;
}

void B200Context::SynchronizeAll()
{
    std::lock_guard<std::mutex> lock(g_ContextsMutex);
    for (B200Context* c : g_Contexts)
    {
        cudaSetDevice(c->m_Device);
        if (c->m_State != State::Capture) { cudaStreamSynchronize(c->m_Stream); }
    }
}

}  // namespace armnn
