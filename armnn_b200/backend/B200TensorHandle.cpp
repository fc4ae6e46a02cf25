#include "B200TensorHandle.hpp"

#include <armnn/Exceptions.hpp>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "b200k.h"

namespace armnn
{

void B200Check(cudaError_t e, const char* what)
{
    if (e != cudaSuccess)
    {
        throw RuntimeException(std::string("B200Acc: ") + what + " failed: " + cudaGetErrorString(e));
    }
}

void B200CheckStatus(int rc)
{
    if (rc != B200K_OK)
    {
        throw RuntimeException(std::string("B200Acc: ") + b200k_last_error());
    }
}

namespace
{
int g_ConfiguredDevice = -1;
std::atomic<uint64_t> g_Epoch{1};
}

uint64_t B200Device::Epoch() { return g_Epoch.load(std::memory_order_relaxed); }
void B200Device::NextEpoch() { g_Epoch.fetch_add(1, std::memory_order_relaxed); }

void B200Device::Configure(int deviceId)
{
    g_ConfiguredDevice = deviceId;
    Get();
}

B200Device::B200Device()
{
    int dev = g_ConfiguredDevice;
    if (dev < 0)
    {
        const char* env = std::getenv("B200ACC_DEVICE_ID");
        dev = env ? std::atoi(env) : 0;
    }
    if (b200k_device_open(dev) != B200K_OK)
    {
        throw BackendUnavailableException(std::string("B200Acc: ") + b200k_last_error());
    }
    m_Device = dev;
    if (cudaStreamCreateWithFlags(&m_Stream, cudaStreamNonBlocking) != cudaSuccess)
    {
        throw BackendUnavailableException("B200Acc: cannot create a CUDA stream");
    }
}

B200Device& B200Device::Get()
{
    static B200Device instance;
    return instance;
}

void B200Device::MakeCurrent() const
{
    B200Check(cudaSetDevice(m_Device), "cudaSetDevice");
}

B200TensorHandle::B200TensorHandle(const TensorInfo& info) : m_Info(info) {}

B200TensorHandle::~B200TensorHandle()
{
    Unimport();
    if (m_Dev) { cudaFree(m_Dev); }
    if (m_Host) { cudaFreeHost(m_Host); }
}

void B200TensorHandle::Allocate()
{
    if (!m_Dev)
    {
        B200Device::Get().MakeCurrent();
        size_t bytes = m_Info.GetNumBytes();
        B200Check(cudaMalloc(&m_Dev, bytes ? bytes : 16), "cudaMalloc");
    }
}

void* B200TensorHandle::Device() const
{
    if (!m_Dev) { const_cast<B200TensorHandle*>(this)->Allocate(); }
    return m_Dev;
}

const void* B200TensorHandle::Map(bool /*blocking*/) const
{
    B200Device& d = B200Device::Get();
    d.MakeCurrent();
    const size_t bytes = m_Info.GetNumBytes();
    if (m_Imported)
    {
        // the user's buffer is the host copy: results go straight into it, inputs are read from it as they are
        m_ReadOnlyMapping = m_DeviceNewer;
        if (m_DeviceNewer)
        {
            PinIfReused();
            B200Check(cudaMemcpyAsync(m_Imported, Device(), bytes, cudaMemcpyDeviceToHost, d.Stream()), "cudaMemcpyAsync D2H");
            m_DeviceNewer = false;
        }
        B200Check(cudaStreamSynchronize(d.Stream()), "cudaStreamSynchronize");
        B200CheckStatus(b200k_poll_status());
        return m_Imported;
    }
    if (!m_Host) { B200Check(cudaMallocHost(&m_Host, bytes ? bytes : 16), "cudaMallocHost"); }
    m_ReadOnlyMapping = m_DeviceNewer;
    if (m_DeviceNewer)
    {
        B200Check(cudaMemcpyAsync(m_Host, Device(), bytes, cudaMemcpyDeviceToHost, d.Stream()), "cudaMemcpyAsync D2H");
        m_DeviceNewer = false;
    }
    // also waits for an earlier Unmap's upload from this staging buffer before the caller overwrites it
    B200Check(cudaStreamSynchronize(d.Stream()), "cudaStreamSynchronize");
    B200CheckStatus(b200k_poll_status());
    return m_Host;
}

void B200TensorHandle::Unmap() const
{
    if (m_Imported)
    {
        if (!m_ReadOnlyMapping) { m_UploadEpoch = 0; }  // the host may have written: upload again before the next read
        return;
    }
    if (!m_Host || m_ReadOnlyMapping) { return; }      // a read-back of device results needs no upload
    B200Device& d = B200Device::Get();
    d.MakeCurrent();
    B200Check(cudaMemcpyAsync(Device(), m_Host, m_Info.GetNumBytes(), cudaMemcpyHostToDevice, d.Stream()), "cudaMemcpyAsync H2D");
}

void B200TensorHandle::CopyOutTo(void* memory) const
{
    B200Device& d = B200Device::Get();
    d.MakeCurrent();
    B200Check(cudaStreamSynchronize(d.Stream()), "cudaStreamSynchronize");
    B200Check(cudaMemcpy(memory, Device(), m_Info.GetNumBytes(), cudaMemcpyDeviceToHost), "cudaMemcpy D2H");
}

void B200TensorHandle::CopyInFrom(const void* memory)
{
    B200Device& d = B200Device::Get();
    d.MakeCurrent();
    B200Check(cudaMemcpyAsync(Device(), memory, m_Info.GetNumBytes(), cudaMemcpyHostToDevice, d.Stream()), "cudaMemcpyAsync H2D");
    B200Check(cudaStreamSynchronize(d.Stream()), "cudaStreamSynchronize");
    m_DeviceNewer = false;
}

bool B200TensorHandle::Import(void* memory, MemorySource source)
{
    if (!CanBeImported(memory, source)) { return false; }
    if (memory != m_Imported)
    {
        Unimport();
        m_Imported = memory;
    }
    m_UploadEpoch = 0;             // new contents: upload before the next read
    m_DeviceNewer = false;
    return true;
}

void B200TensorHandle::Unimport()
{
    if (m_Imported && m_Registered)
    {
        cudaStreamSynchronize(B200Device::Get().Stream());
        if (cudaHostUnregister(m_Imported) != cudaSuccess) { cudaGetLastError(); }
    }
    m_Imported = nullptr;
    m_Registered = false;
    m_Transfers = 0;
}

// A buffer that serves a second inference (imported again with the same address, or pre-imported once through
// IRuntime::ImportInputs / ImportOutputs) is page-locked, so that this and every later transfer is an asynchronous DMA
// at full PCIe rate; the first transfer of a buffer goes through the driver's own staging.  Memory the user has
// pinned already reports an error here, which is just as good.
void B200TensorHandle::PinIfReused() const
{
    if (m_Transfers++ == 0 || m_Registered || m_Transfers > 2) { return; }
    const size_t bytes = m_Info.GetNumBytes();
    m_Registered = cudaHostRegister(m_Imported, bytes ? bytes : 16, cudaHostRegisterDefault) == cudaSuccess;
    if (!m_Registered) { cudaGetLastError(); }
}

void B200TensorHandle::SyncImportedToDevice() const
{
    if (!m_Imported || m_DeviceNewer) { return; }       // not imported, or produced on the device in this inference
    const uint64_t epoch = B200Device::Epoch();
    if (m_UploadEpoch == epoch) { return; }
    B200Device& d = B200Device::Get();
    d.MakeCurrent();
    PinIfReused();
    B200Check(cudaMemcpyAsync(Device(), m_Imported, m_Info.GetNumBytes(), cudaMemcpyHostToDevice, d.Stream()), "cudaMemcpyAsync H2D");
    m_UploadEpoch = epoch;
}

const ITensorHandleFactory::FactoryId& B200TensorHandleFactory::GetIdStatic()
{
    static const FactoryId s_Id(B200TensorHandleFactoryId());
    return s_Id;
}

}  // namespace armnn
