#include "B200TensorHandle.hpp"

#include <armnn/Exceptions.hpp>

#include <cstring>
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

// ---- memory manager ------------------------------------------------------------------------------------------

B200MemoryManager::~B200MemoryManager()
{
    if (m_Arena)
    {
        if (m_Ctx) { cudaSetDevice(m_Ctx->Device()); }
        cudaFree(m_Arena);
    }
}

B200MemoryManager::Pool* B200MemoryManager::Manage(size_t bytes)
{
    if (m_Arena) { throw RuntimeException("B200Acc: tensor lifetimes cannot change while the arena is acquired"); }
    m_ManagedBytes += bytes;
    // the smallest free pool that is large enough; otherwise the largest free one grows; otherwise a new pool
    Pool* best = nullptr;
    Pool* largest = nullptr;
    for (auto& p : m_Pools)
    {
        if (!p->free) { continue; }
        if (p->bytes >= bytes && (!best || p->bytes < best->bytes)) { best = p.get(); }
        if (!largest || p->bytes > largest->bytes) { largest = p.get(); }
    }
    Pool* pool = best ? best : largest;
    if (!pool)
    {
        m_Pools.push_back(std::make_unique<Pool>());
        pool = m_Pools.back().get();
    }
    if (pool->bytes < bytes) { pool->bytes = bytes; }
    pool->free = false;
    return pool;
}

void B200MemoryManager::Allocate(Pool* pool)
{
    if (pool) { pool->free = true; }
}

void B200MemoryManager::Acquire()
{
    if (m_Arena) { return; }
    size_t total = 0;
    for (auto& p : m_Pools)
    {
        p->offset = total;
        total += (p->bytes + 255) & ~static_cast<size_t>(255);
    }
    m_ArenaBytes = total;
    if (total == 0) { return; }
    if (m_Ctx) { m_Ctx->MakeCurrent(); }
    B200Check(cudaMalloc(&m_Arena, total), "cudaMalloc (tensor arena)");
}

void B200MemoryManager::Release()
{
    if (!m_Arena) { return; }
    if (m_Ctx)
    {
        m_Ctx->MakeCurrent();
        m_Ctx->Invalidate();                          // a recorded graph holds addresses inside the arena
        cudaStreamSynchronize(m_Ctx->Stream());
    }
    cudaFree(m_Arena);
    m_Arena = nullptr;
}

void* B200MemoryManager::Address(const Pool* pool)
{
    if (!m_Arena) { Acquire(); }
    return static_cast<char*>(m_Arena) + pool->offset;
}

// ---- tensor handle -------------------------------------------------------------------------------------------

B200TensorHandle::B200TensorHandle(const TensorInfo& info, std::shared_ptr<B200Context> ctx, std::shared_ptr<B200MemoryManager> mgr)
    : m_Info(info), m_Ctx(std::move(ctx)), m_Mgr(std::move(mgr)) {}

B200TensorHandle::~B200TensorHandle()
{
    Unimport();
    if (m_Dev || m_Host) { cudaSetDevice(m_Ctx->Device()); }
    if (m_Dev) { cudaFree(m_Dev); }
    if (m_Host) { cudaFreeHost(m_Host); }
}

void B200TensorHandle::Manage()
{
    // start of this tensor's lifetime in the network's execution order
    if (m_Mgr && !m_Pool && !m_Dev) { m_Pool = m_Mgr->Manage(m_Info.GetNumBytes() ? m_Info.GetNumBytes() : 16); }
}

void B200TensorHandle::Allocate()
{
    if (m_Pool)
    {
        m_Mgr->Allocate(m_Pool);                       // end of the lifetime: the bytes may serve a later tensor
        return;
    }
    if (!m_Dev)
    {
        m_Ctx->MakeCurrent();
        size_t bytes = m_Info.GetNumBytes();
        B200Check(cudaMalloc(&m_Dev, bytes ? bytes : 16), "cudaMalloc");
    }
}

void* B200TensorHandle::Device() const
{
    if (m_Pool) { return m_Mgr->Address(m_Pool); }
    if (!m_Dev) { const_cast<B200TensorHandle*>(this)->Allocate(); }
    return m_Dev;
}

const void* B200TensorHandle::Map(bool /*blocking*/) const
{
    B200Context& d = *m_Ctx;
    d.MakeCurrent();
    const size_t bytes = m_Info.GetNumBytes();
    if (m_Imported)
    {
        // the user's buffer is the host copy: results go straight into it, inputs are read from it as they are
        m_ReadOnlyMapping = m_DeviceNewer;
        if (m_DeviceNewer)
        {
            d.SyncForMap();                            // (ends a recording, if one is running, before the copy is enqueued)
            PinIfReused();
            B200Check(cudaMemcpyAsync(m_Imported, Device(), bytes, cudaMemcpyDeviceToHost, d.Stream()), "cudaMemcpyAsync D2H");
            m_DeviceNewer = false;
        }
        d.SyncForMap();
        B200CheckStatus(b200k_poll_status());
        return m_Imported;
    }
    if (!m_Host) { B200Check(cudaMallocHost(&m_Host, bytes ? bytes : 16), "cudaMallocHost"); }
    m_ReadOnlyMapping = m_DeviceNewer;
    if (m_DeviceNewer)
    {
        d.SyncForMap();
        B200Check(cudaMemcpyAsync(m_Host, Device(), bytes, cudaMemcpyDeviceToHost, d.Stream()), "cudaMemcpyAsync D2H");
        m_DeviceNewer = false;
    }
    // also waits for an earlier Unmap's upload from this staging buffer before the caller overwrites it
    d.SyncForMap();
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
    m_Ctx->MakeCurrent();
    B200Check(cudaMemcpyAsync(Device(), m_Host, m_Info.GetNumBytes(), cudaMemcpyHostToDevice, m_Ctx->Stream()), "cudaMemcpyAsync H2D");
}

void B200TensorHandle::CopyOutTo(void* memory) const
{
    m_Ctx->SyncForMap();
    B200Check(cudaMemcpy(memory, Device(), m_Info.GetNumBytes(), cudaMemcpyDeviceToHost), "cudaMemcpy D2H");
}

void B200TensorHandle::CopyInFrom(const void* memory)
{
    m_Ctx->SyncForMap();
    B200Check(cudaMemcpyAsync(Device(), memory, m_Info.GetNumBytes(), cudaMemcpyHostToDevice, m_Ctx->Stream()), "cudaMemcpyAsync H2D");
    B200Check(cudaStreamSynchronize(m_Ctx->Stream()), "cudaStreamSynchronize");
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
        cudaSetDevice(m_Ctx->Device());
        cudaStreamSynchronize(m_Ctx->Stream());
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
    const uint64_t epoch = m_Ctx->Epoch();
    if (m_UploadEpoch == epoch) { return; }
    m_Ctx->MakeCurrent();
    PinIfReused();
    B200Check(cudaMemcpyAsync(Device(), m_Imported, m_Info.GetNumBytes(), cudaMemcpyHostToDevice, m_Ctx->Stream()), "cudaMemcpyAsync H2D");
    m_UploadEpoch = epoch;
}

// ---- factory -------------------------------------------------------------------------------------------------

const ITensorHandleFactory::FactoryId& B200TensorHandleFactory::GetIdStatic()
{
    static const FactoryId s_Id(B200TensorHandleFactoryId());
    return s_Id;
}

std::shared_ptr<B200Context> B200TensorHandleFactory::Ctx() const
{
    if (!m_Ctx) { m_Ctx = B200Context::Shared(); }
    return m_Ctx;
}

std::unique_ptr<ITensorHandle> B200TensorHandleFactory::Create(const TensorInfo& info, bool managed) const
{
    return std::make_unique<B200TensorHandle>(info, Ctx(), managed ? m_MemoryManager : nullptr);
}

}  // namespace armnn
