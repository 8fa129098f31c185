// Passing open file descriptors between the processes of one node.
//
// The cuMem VMM backend of the symmetric memory (symm_vmm.cc) exports every physical allocation as a POSIX file
// descriptor. A descriptor is only a number inside its own process; another process gets a working duplicate through
// an SCM_RIGHTS control message on a Unix-domain socket. Each process that has something to export runs ONE small
// server thread on the abstract socket "\0coccl-fd-<pid>"; an importer connects, sends the 64-bit key of what it
// wants, and receives the descriptor. Keys are chosen by the exporter and travel to the importers inside the
// (plain-bytes) export handles.
//
// NCCL does the same for its cuMem handles through its proxy service's Unix socket (src/misc/ipcsocket.cc,
// src/proxy.cc `ncclProxyMsgGetFd`); the reference inherits that path for its VMM workspace
// (src/coccl-extend/core/memory/coccl_buffer_vmm.cc:152-240 maps within one process only).
#pragma once
#include <stdint.h>

namespace coccl {

// Make descriptor `fd` obtainable by other processes under `key` (the server thread starts at the first call).
// The channel keeps its own duplicate, so the caller may close `fd` afterwards. Returns 0 or an errno value.
int fdChannelPublish(uint64_t key, int fd);
// Stop offering `key` and close the channel's duplicate.
void fdChannelWithdraw(uint64_t key);
// Obtain a duplicate of the descriptor that process `pid` published under `key`. Returns the new descriptor
// (the caller closes it) or -errno. Works for the calling process's own pid too.
int fdChannelFetch(int pid, uint64_t key, int timeoutMs);
// Stop the server thread and close every published duplicate (tests; otherwise it lives as long as the process).
void fdChannelShutdown();

}  // namespace coccl
