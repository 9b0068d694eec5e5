// Peer-visible arenas (CUDA IPC) and host-mapped status words.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>

#include "lbc_api.h"

namespace lbc {

struct StatusWord {
    uintptr_t host;    // CPU address of the pinned LbcStatus
    uintptr_t device;  // address kernels use for the same memory
};

uintptr_t arena_alloc(size_t nbytes);           // zero-filled cudaMalloc on the current device
void arena_free(uintptr_t ptr);
std::string ipc_get_handle(uintptr_t ptr);      // 64 opaque bytes, send to the peers
uintptr_t ipc_open_handle(const std::string& bytes);
void ipc_close_handle(uintptr_t ptr);
bool can_access_peer(int device, int peer);
void enable_peer_access(int peer);
StatusWord status_alloc();
void status_free(uintptr_t host);
LbcStatus status_read(uintptr_t host);
void status_clear(uintptr_t host);

}  // namespace lbc
