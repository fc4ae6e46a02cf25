// Device-memory tensor handles of the B200Acc backend, their factory and memory manager, and the per-process
// device context (device id + the CUDA stream every workload is enqueued on).
//
// Arm NN moves network inputs and outputs with CopyMemGenericWorkload, which Map()s both handles and memcpy()s
// (src/backends/backendsCommon/MemCopyWorkload.cpp:51-64), so a device handle owns a pinned host staging buffer:
// Map() = stream synchronise + device->host copy when the device copy is newer, Unmap() = host->device copy.
// The blocking Map of the output handle is the only per-inference synchronisation point.
//
// With INetworkProperties{MemorySource::Malloc, MemorySource::Malloc} (or IRuntime::ImportInputs / ImportOutputs) the
// core hands the user's own buffers to Import() instead (src/armnn/LoadedNetwork.cpp:1008-1030, 1086-1115, 1401-1520):
// an imported handle has no staging buffer; its device copy is filled straight from the user's memory when the first
// workload of an inference reads it, and a handle a workload has written is copied straight into the user's memory
// by the Map() of the core's SyncMemGenericWorkload.  A buffer that comes back for a second inference is page-locked
// (cudaHostRegister) until Unimport(), so that its transfers are asynchronous DMA.
#pragma once

#include <armnn/backends/IMemoryManager.hpp>
#include <armnn/backends/ITensorHandle.hpp>
#include <armnn/backends/ITensorHandleFactory.hpp>
#include <armnn/backends/TensorHandle.hpp>

#include <cuda_runtime.h>

#include <cstdint>

namespace armnn
{

constexpr const char* B200BackendId() { return "B200Acc"; }
constexpr const char* B200TensorHandleFactoryId() { return "Nv/B200Acc/TensorHandleFactory"; }

/// Device id and stream shared by every handle and workload of this process (one process drives one GPU;
/// the device comes from the "DeviceId" backend option, or B200ACC_DEVICE_ID, or 0).
class B200Device
{
public:
    static B200Device& Get();
    static void Configure(int deviceId);            // before first use; throws BackendUnavailableException
    cudaStream_t Stream() const { return m_Stream; }
    /// Counts inferences (advanced by IBackendContext::AfterEnqueueWorkload): an imported input is uploaded once per epoch.
    static uint64_t Epoch();
    static void NextEpoch();
    int Id() const { return m_Device; }
    void MakeCurrent() const;
private:
    B200Device();
    int m_Device = 0;
    cudaStream_t m_Stream = nullptr;
};

void B200Check(cudaError_t e, const char* what);     // throws armnn::RuntimeException
void B200CheckStatus(int rc);                        // libb200k status -> armnn::RuntimeException

class B200MemoryManager : public IMemoryManager
{
public:
    void Acquire() override {}                       // handles own their device buffers (see Allocate)
    void Release() override {}
};

class B200TensorHandle : public ITensorHandle
{
public:
    explicit B200TensorHandle(const TensorInfo& info);
    ~B200TensorHandle() override;

    void Manage() override {}
    void Allocate() override;
    ITensorHandle* GetParent() const override { return nullptr; }

    const void* Map(bool blocking = true) const override;
    using ITensorHandle::Map;
    void Unmap() const override;

    TensorShape GetStrides() const override { return GetUnpaddedTensorStrides(m_Info); }
    TensorShape GetShape() const override { return m_Info.GetShape(); }
    const TensorInfo& GetTensorInfo() const { return m_Info; }

    void CopyOutTo(void* memory) const override;
    void CopyInFrom(const void* memory) override;

    unsigned int GetImportFlags() const override { return static_cast<unsigned int>(MemorySource::Malloc); }
    bool CanBeImported(void* memory, MemorySource source) override { return memory != nullptr && source == MemorySource::Malloc; }
    bool Import(void* memory, MemorySource source) override;
    void Unimport() override;
    /// For a workload about to read this handle: when it is an imported network input, bring the user's memory to
    /// the device (once per inference).
    void SyncImportedToDevice() const;

    /// Device pointer for kernels (allocates on first use).
    void* Device() const;
    /// A workload has written the device copy: the next Map() must read it back.
    void MarkDeviceWritten() const { m_DeviceNewer = true; }

private:
    B200TensorHandle(const B200TensorHandle&) = delete;
    B200TensorHandle& operator=(const B200TensorHandle&) = delete;

    TensorInfo m_Info;
    mutable void* m_Dev = nullptr;
    mutable void* m_Host = nullptr;                  // pinned staging
    mutable bool m_DeviceNewer = false;
    mutable bool m_ReadOnlyMapping = false;
    void PinIfReused() const;
    void* m_Imported = nullptr;                      // the user's buffer (host), or nullptr
    mutable bool m_Registered = false;               // we page-locked m_Imported
    mutable unsigned int m_Transfers = 0;            // transfers from / to m_Imported so far
    mutable uint64_t m_UploadEpoch = 0;
};

class B200TensorHandleFactory : public ITensorHandleFactory
{
public:
    explicit B200TensorHandleFactory(std::shared_ptr<B200MemoryManager> mgr) : m_MemoryManager(std::move(mgr)) {}

    std::unique_ptr<ITensorHandle> CreateSubTensorHandle(ITensorHandle&, TensorShape const&, unsigned int const*) const override
    { return nullptr; }
    std::unique_ptr<ITensorHandle> CreateTensorHandle(const TensorInfo& info) const override
    { return std::make_unique<B200TensorHandle>(info); }
    std::unique_ptr<ITensorHandle> CreateTensorHandle(const TensorInfo& info, DataLayout) const override
    { return std::make_unique<B200TensorHandle>(info); }
    std::unique_ptr<ITensorHandle> CreateTensorHandle(const TensorInfo& info, const bool) const override
    { return std::make_unique<B200TensorHandle>(info); }
    std::unique_ptr<ITensorHandle> CreateTensorHandle(const TensorInfo& info, DataLayout, const bool) const override
    { return std::make_unique<B200TensorHandle>(info); }

    static const FactoryId& GetIdStatic();
    const FactoryId& GetId() const override { return GetIdStatic(); }
    bool SupportsSubTensors() const override { return false; }
    bool SupportsMapUnmap() const override { return true; }
    MemorySourceFlags GetExportFlags() const override { return 0; }
    MemorySourceFlags GetImportFlags() const override { return static_cast<MemorySourceFlags>(MemorySource::Malloc); }

private:
    std::shared_ptr<B200MemoryManager> m_MemoryManager;
};

}  // namespace armnn
