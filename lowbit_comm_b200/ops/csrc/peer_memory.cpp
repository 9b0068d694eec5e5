// Peer-visible device memory for one-process-per-GPU jobs on a single NVLink
// domain: raw cudaMalloc arenas exported with CUDA IPC handles, mapped by every
// other rank, plus pinned host status words that a kernel can write and the
// host can read without synchronising.
//
// The reference has no counterpart: it moves payloads with torch.distributed
// calls (ccdl_comm/communication/torch_transport.py:61-188) and never maps
// another GPU's memory.
#include "peer_memory.h"

#include <cuda_runtime.h>

#include <cstring>
#include <stdexcept>
#include <string>

namespace lbc {

static void check(cudaError_t err, const char* what) {
    if (err != cudaSuccess) {
        // clear the sticky-free error so later calls start clean
        cudaGetLastError();
        throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(err));
    }
}

uintptr_t arena_alloc(size_t nbytes) {
    void* ptr = nullptr;
    check(cudaMalloc(&ptr, nbytes), "cudaMalloc(arena)");
    check(cudaMemset(ptr, 0, nbytes), "cudaMemset(arena)");
    check(cudaDeviceSynchronize(), "cudaDeviceSynchronize(arena)");
    return reinterpret_cast<uintptr_t>(ptr);
}

void arena_free(uintptr_t ptr) { check(cudaFree(reinterpret_cast<void*>(ptr)), "cudaFree(arena)"); }

std::string ipc_get_handle(uintptr_t ptr) {
    cudaIpcMemHandle_t handle;
    check(cudaIpcGetMemHandle(&handle, reinterpret_cast<void*>(ptr)), "cudaIpcGetMemHandle");
    return std::string(reinterpret_cast<const char*>(&handle), sizeof(handle));
}

uintptr_t ipc_open_handle(const std::string& bytes) {
    if (bytes.size() != sizeof(cudaIpcMemHandle_t)) throw std::runtime_error("bad IPC handle size");
    cudaIpcMemHandle_t handle;
    std::memcpy(&handle, bytes.data(), sizeof(handle));
    void* ptr = nullptr;
    check(cudaIpcOpenMemHandle(&ptr, handle, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    return reinterpret_cast<uintptr_t>(ptr);
}

void ipc_close_handle(uintptr_t ptr) { check(cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)), "cudaIpcCloseMemHandle"); }

bool can_access_peer(int device, int peer) {
    if (device == peer) return true;
    int ok = 0;
    check(cudaDeviceCanAccessPeer(&ok, device, peer), "cudaDeviceCanAccessPeer");
    return ok != 0;
}

void enable_peer_access(int peer) {
    cudaError_t err = cudaDeviceEnablePeerAccess(peer, 0);
    if (err == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();
        return;
    }
    check(err, "cudaDeviceEnablePeerAccess");
}

StatusWord status_alloc() {
    void* host = nullptr;
    check(cudaHostAlloc(&host, sizeof(LbcStatus), cudaHostAllocMapped | cudaHostAllocPortable), "cudaHostAlloc(status)");
    std::memset(host, 0, sizeof(LbcStatus));
    void* dev = nullptr;
    check(cudaHostGetDevicePointer(&dev, host, 0), "cudaHostGetDevicePointer(status)");
    return StatusWord{reinterpret_cast<uintptr_t>(host), reinterpret_cast<uintptr_t>(dev)};
}

void status_free(uintptr_t host) { check(cudaFreeHost(reinterpret_cast<void*>(host)), "cudaFreeHost(status)"); }

LbcStatus status_read(uintptr_t host) {
    LbcStatus out;
    std::memcpy(&out, reinterpret_cast<const void*>(host), sizeof(out));
    return out;
}

void status_clear(uintptr_t host) { std::memset(reinterpret_cast<void*>(host), 0, sizeof(LbcStatus)); }

}  // namespace lbc
