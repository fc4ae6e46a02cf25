// CudaEventTimer: the device-time instrument of B200Acc workloads for the Arm NN profiler, the counterpart of
// OpenClTimer (src/backends/cl/OpenClTimer.hpp:20-60 of the Arm NN tree).  A workload opens
//     ARMNN_SCOPED_PROFILING_EVENT_WITH_INSTRUMENTS(backend, guid, name, WallClockTimer(), CudaEventTimer(stream))
// around its launches; with profiling enabled (INetworkProperties::m_ProfilingEnabled) the event then carries the wall
// clock of Execute() on the host and the time the workload's kernels took on the GPU (CUDA events recorded on the
// network's stream before and after the launches).  Nothing is created or recorded unless the profiler is enabled:
// ScopedProfilingEvent only calls Start() / Stop() on an enabled profiler.
#pragma once

#include <Instrument.hpp>

#include <cuda_runtime.h>

#include <vector>

namespace armnn
{

class CudaEventTimer : public Instrument
{
public:
    explicit CudaEventTimer(cudaStream_t stream, int device) : m_Stream(stream), m_Device(device) {}
    CudaEventTimer(CudaEventTimer&& o) noexcept
        : m_Stream(o.m_Stream), m_Device(o.m_Device), m_Start(o.m_Start), m_Stop(o.m_Stop) { o.m_Start = o.m_Stop = nullptr; }
    CudaEventTimer(const CudaEventTimer&) = delete;
    CudaEventTimer& operator=(const CudaEventTimer&) = delete;
    ~CudaEventTimer() override
    {
        if (m_Start) { cudaEventDestroy(m_Start); }
        if (m_Stop) { cudaEventDestroy(m_Stop); }
    }

    void Start() override
    {
        cudaSetDevice(m_Device);
        if (!m_Start && cudaEventCreate(&m_Start) != cudaSuccess) { m_Start = nullptr; }
        if (!m_Stop && cudaEventCreate(&m_Stop) != cudaSuccess) { m_Stop = nullptr; }
        if (m_Start) { cudaEventRecord(m_Start, m_Stream); }
    }

    void Stop() override
    {
        if (m_Stop) { cudaEventRecord(m_Stop, m_Stream); }
    }

    bool HasKernelMeasurements() const override { return true; }

    const char* GetName() const override { return "CudaEventTimer"; }

    /// Device time between Start() and Stop() on the workload's stream; waits for the stop event.
    std::vector<Measurement> GetMeasurements() const override
    {
        std::vector<Measurement> out;
        float ms = 0.f;
        if (m_Start && m_Stop && cudaEventSynchronize(m_Stop) == cudaSuccess &&
            cudaEventElapsedTime(&ms, m_Start, m_Stop) == cudaSuccess)
        {
            out.emplace_back("B200 kernel time", static_cast<double>(ms) * 1000.0, Measurement::Unit::TIME_US);
        }
        return out;
    }

private:
    cudaStream_t m_Stream;
    int m_Device;
    cudaEvent_t m_Start = nullptr, m_Stop = nullptr;
};

}  // namespace armnn
