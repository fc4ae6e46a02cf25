// Device-memory tensor handles of the B200Acc backend, their factory and memory manager, and the per-process
// device context (device id + the CUDA stream every workload is enqueued on).
//
// Arm NN moves network inputs and outputs with CopyMemGenericWorkload, which Map()s both handles and memcpy()s
// (src/backends/backendsCommon/MemCopyWorkload.cpp:51-64), so a device handle owns a pinned host staging buffer:
// Map() = stream synchronise + device->host copy when the device copy is newer, Unmap() = host->device copy.
// The blocking Map of the output handle is the only per-inference synchronisation point.
#pragma once

#include <armnn/backends/IMemoryManager.hpp>
#include <armnn/backends/ITensorHandle.hpp>
#include <armnn/backends/ITensorHandleFactory.hpp>
#include <armnn/backends/TensorHandle.hpp>

#include <cuda_runtime.h>

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
    MemorySourceFlags GetImportFlags() const override { return 0; }

private:
    std::shared_ptr<B200MemoryManager> m_MemoryManager;
};

}  // namespace armnn
