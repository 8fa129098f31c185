#include "symm/fd_channel.h"

#include <errno.h>
#include <fcntl.h>
#include <poll.h>
#include <stddef.h>
#include <stdio.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <map>
#include <mutex>
#include <thread>

namespace coccl {
namespace {

struct Channel {
  std::mutex mutex;
  std::map<uint64_t, int> published;  // key -> this channel's duplicate of the descriptor
  int listenFd = -1;
  int wakePipe[2] = {-1, -1};
  std::thread server;
  bool running = false;
};

Channel& channel() {
  static Channel* c = new Channel();  // never destroyed: the server thread may outlive static destructors
  return *c;
}

// Abstract-namespace address: no file system entry, gone with the process.
socklen_t addressOf(int pid, sockaddr_un* addr) {
  memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  const int n = snprintf(addr->sun_path + 1, sizeof(addr->sun_path) - 1, "coccl-fd-%d", pid);
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + (size_t)n);
}

int sendFd(int sock, int fd, int32_t status) {
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  iovec iov{&status, sizeof(status)};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
  if (fd >= 0) {
    memset(control, 0, sizeof(control));
    msg.msg_control = control;
    msg.msg_controllen = sizeof(control);
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(c), &fd, sizeof(int));
  }
  return sendmsg(sock, &msg, MSG_NOSIGNAL) == (ssize_t)sizeof(status) ? 0 : errno;
}

int recvFd(int sock, int* fd) {
  *fd = -1;
  int32_t status = 0;
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  iovec iov{&status, sizeof(status)};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
  memset(control, 0, sizeof(control));
  msg.msg_control = control;
  msg.msg_controllen = sizeof(control);
  const ssize_t got = recvmsg(sock, &msg, MSG_CMSG_CLOEXEC);
  if (got != (ssize_t)sizeof(status)) return got < 0 ? errno : EPROTO;
  if (status != 0) return status;
  for (cmsghdr* c = CMSG_FIRSTHDR(&msg); c != nullptr; c = CMSG_NXTHDR(&msg, c)) {
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS && c->cmsg_len >= CMSG_LEN(sizeof(int))) {
      memcpy(fd, CMSG_DATA(c), sizeof(int));
      return 0;
    }
  }
  return EPROTO;
}

void serve(Channel* c) {
  for (;;) {
    pollfd fds[2] = {{c->listenFd, POLLIN, 0}, {c->wakePipe[0], POLLIN, 0}};
    if (poll(fds, 2, -1) < 0) {
      if (errno == EINTR) continue;
      return;
    }
    if (fds[1].revents != 0) return;  // shutdown
    if ((fds[0].revents & POLLIN) == 0) continue;
    const int conn = accept(c->listenFd, nullptr, nullptr);
    if (conn < 0) continue;
    // one request per connection: the key; a client that sends nothing within a second is dropped
    pollfd one{conn, POLLIN, 0};
    uint64_t key = 0;
    if (poll(&one, 1, 1000) == 1 && recv(conn, &key, sizeof(key), MSG_WAITALL) == (ssize_t)sizeof(key)) {
      int fd = -1;
      {
        std::lock_guard<std::mutex> lock(c->mutex);
        auto it = c->published.find(key);
        if (it != c->published.end()) fd = it->second;
        // sendmsg duplicates the descriptor into the message while the lock is held, so a concurrent withdraw
        // cannot close it in between
        sendFd(conn, fd, fd >= 0 ? 0 : ENOENT);
      }
    }
    close(conn);
  }
}

int startLocked(Channel& c) {
  if (c.running) return 0;
  c.listenFd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (c.listenFd < 0) return errno;
  sockaddr_un addr;
  const socklen_t len = addressOf((int)getpid(), &addr);
  if (bind(c.listenFd, reinterpret_cast<sockaddr*>(&addr), len) != 0 || listen(c.listenFd, 64) != 0 || pipe(c.wakePipe) != 0) {
    const int e = errno;
    close(c.listenFd);
    c.listenFd = -1;
    return e;
  }
  c.running = true;
  c.server = std::thread(serve, &c);
  return 0;
}

}  // namespace

int fdChannelPublish(uint64_t key, int fd) {
  Channel& c = channel();
  std::lock_guard<std::mutex> lock(c.mutex);
  const int rc = startLocked(c);
  if (rc != 0) return rc;
  const int dup = fcntl(fd, F_DUPFD_CLOEXEC, 0);
  if (dup < 0) return errno;
  auto it = c.published.find(key);
  if (it != c.published.end()) close(it->second);
  c.published[key] = dup;
  return 0;
}

void fdChannelWithdraw(uint64_t key) {
  Channel& c = channel();
  std::lock_guard<std::mutex> lock(c.mutex);
  auto it = c.published.find(key);
  if (it == c.published.end()) return;
  close(it->second);
  c.published.erase(it);
}

int fdChannelFetch(int pid, uint64_t key, int timeoutMs) {
  const int sock = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (sock < 0) return -errno;
  sockaddr_un addr;
  const socklen_t len = addressOf(pid, &addr);
  // the exporter publishes before it hands out the handle, so its server is listening by the time anyone fetches
  if (connect(sock, reinterpret_cast<sockaddr*>(&addr), len) != 0) { const int e = errno; close(sock); return -e; }
  int result = -EPROTO;
  if (send(sock, &key, sizeof(key), MSG_NOSIGNAL) == (ssize_t)sizeof(key)) {
    pollfd one{sock, POLLIN, 0};
    const int ready = poll(&one, 1, timeoutMs);
    if (ready == 1) {
      int fd = -1;
      const int rc = recvFd(sock, &fd);
      result = rc == 0 ? fd : -rc;
    } else {
      result = ready == 0 ? -ETIMEDOUT : -errno;
    }
  } else {
    result = -errno;
  }
  close(sock);
  return result;
}

void fdChannelShutdown() {
  Channel& c = channel();
  std::thread server;
  {
    std::lock_guard<std::mutex> lock(c.mutex);
    if (!c.running) return;
    const char b = 1;
    if (write(c.wakePipe[1], &b, 1) != 1) { /* the poll also ends when the pipe closes below */ }
    server = std::move(c.server);
  }
  if (server.joinable()) server.join();
  std::lock_guard<std::mutex> lock(c.mutex);
  for (auto& kv : c.published) close(kv.second);
  c.published.clear();
  close(c.listenFd);
  close(c.wakePipe[0]);
  close(c.wakePipe[1]);
  c.listenFd = c.wakePipe[0] = c.wakePipe[1] = -1;
  c.running = false;
}

}  // namespace coccl
