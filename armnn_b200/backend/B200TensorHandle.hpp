// Device-memory tensor handles of the B200Acc backend, their factory and memory manager.
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
//
// Device memory.  Handles created as "memory managed" take part in the Manage() / Allocate() lifetime protocol of the
// core (src/armnn/Network.cpp and LoadedNetwork.cpp call Manage() when a tensor is first produced and Allocate() once
// its last consumer has been created): B200MemoryManager packs them into one device arena in which tensors whose
// lifetimes do not overlap share bytes, the scheme of RefMemoryManager (src/backends/reference/RefMemoryManager.cpp:
// 20-103).  All other handles (network inputs and outputs, constants) own their device buffer.
#pragma once

#include <armnn/backends/IMemoryManager.hpp>
#include <armnn/backends/ITensorHandle.hpp>
#include <armnn/backends/ITensorHandleFactory.hpp>
#include <armnn/backends/TensorHandle.hpp>

#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <vector>

#include "B200Context.hpp"

namespace armnn
{

constexpr const char* B200BackendId() { return "B200Acc"; }
constexpr const char* B200TensorHandleFactoryId() { return "Nv/B200Acc/TensorHandleFactory"; }

void B200Check(cudaError_t e, const char* what);     // throws armnn::RuntimeException
void B200CheckStatus(int rc);                        // libb200k status -> armnn::RuntimeException

/// One device arena per network.  Between Manage() and Allocate() a tensor is "live"; a pool (a byte range of the
/// arena) serves one live tensor at a time and is handed to the next tensor that fits once its user called Allocate().
/// Acquire() gives the arena device memory, Release() takes it away (IMemoryManager, driven by
/// LoadedNetwork::AllocateWorkingMemory / FreeWorkingMemory, src/armnn/LoadedNetwork.cpp:1186-1222).
class B200MemoryManager : public IMemoryManager
{
public:
    struct Pool
    {
        size_t bytes = 0;
        size_t offset = 0;                           // inside the arena
        bool free = false;
    };

    explicit B200MemoryManager(std::shared_ptr<B200Context> ctx = nullptr) : m_Ctx(std::move(ctx)) {}
    ~B200MemoryManager() override;

    Pool* Manage(size_t bytes);                      // start of a tensor's lifetime: a pool of at least `bytes`
    void Allocate(Pool* pool);                       // end of its lifetime: the pool may serve a later tensor
    void* Address(const Pool* pool);                 // device address (acquires the arena on first use)

    void Acquire() override;
    void Release() override;

    size_t ArenaBytes() const { return m_ArenaBytes; }
    size_t ManagedBytes() const { return m_ManagedBytes; }   // sum of all managed tensors (what separate buffers would take)

private:
    std::shared_ptr<B200Context> m_Ctx;
    std::vector<std::unique_ptr<Pool>> m_Pools;
    size_t m_ArenaBytes = 0, m_ManagedBytes = 0;
    void* m_Arena = nullptr;
};

class B200TensorHandle : public ITensorHandle
{
public:
    B200TensorHandle(const TensorInfo& info, std::shared_ptr<B200Context> ctx, std::shared_ptr<B200MemoryManager> mgr = nullptr);
    ~B200TensorHandle() override;

    void Manage() override;
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
    bool IsImported() const { return m_Imported != nullptr; }
    /// For a workload about to read this handle: when it is an imported network input, bring the user's memory to
    /// the device (once per inference).
    void SyncImportedToDevice() const;

    /// Device pointer for kernels (allocates on first use).
    void* Device() const;
    /// A workload has written the device copy: the next Map() must read it back.
    void MarkDeviceWritten() const { m_DeviceNewer = true; }
    B200Context& Context() const { return *m_Ctx; }

private:
    B200TensorHandle(const B200TensorHandle&) = delete;
    B200TensorHandle& operator=(const B200TensorHandle&) = delete;

    TensorInfo m_Info;
    std::shared_ptr<B200Context> m_Ctx;
    std::shared_ptr<B200MemoryManager> m_Mgr;        // null: the handle owns its buffer
    B200MemoryManager::Pool* m_Pool = nullptr;
    mutable void* m_Dev = nullptr;                   // own buffer (unmanaged handles)
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
    B200TensorHandleFactory(std::shared_ptr<B200Context> ctx, std::shared_ptr<B200MemoryManager> mgr)
        : m_Ctx(std::move(ctx)), m_MemoryManager(std::move(mgr)) {}

    std::unique_ptr<ITensorHandle> CreateSubTensorHandle(ITensorHandle&, TensorShape const&, unsigned int const*) const override
    { return nullptr; }
    std::unique_ptr<ITensorHandle> CreateTensorHandle(const TensorInfo& info) const override
    { return Create(info, true); }
    std::unique_ptr<ITensorHandle> CreateTensorHandle(const TensorInfo& info, DataLayout) const override
    { return Create(info, true); }
    std::unique_ptr<ITensorHandle> CreateTensorHandle(const TensorInfo& info, const bool isMemoryManaged) const override
    { return Create(info, isMemoryManaged); }
    std::unique_ptr<ITensorHandle> CreateTensorHandle(const TensorInfo& info, DataLayout, const bool isMemoryManaged) const override
    { return Create(info, isMemoryManaged); }

    static const FactoryId& GetIdStatic();
    const FactoryId& GetId() const override { return GetIdStatic(); }
    bool SupportsSubTensors() const override { return false; }
    bool SupportsMapUnmap() const override { return true; }
    MemorySourceFlags GetExportFlags() const override { return 0; }
    MemorySourceFlags GetImportFlags() const override { return static_cast<MemorySourceFlags>(MemorySource::Malloc); }

private:
    std::unique_ptr<ITensorHandle> Create(const TensorInfo& info, bool managed) const;
    /// The optimizer also creates factories (to pick handle strategies) long before any device is needed: the context is
    /// made on first use.
    std::shared_ptr<B200Context> Ctx() const;
    mutable std::shared_ptr<B200Context> m_Ctx;
    std::shared_ptr<B200MemoryManager> m_MemoryManager;
};

}  // namespace armnn
