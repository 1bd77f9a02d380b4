// All-to-all exchange of POSIX file descriptors between the ranks of one node over
// AF_UNIX datagram sockets (SCM_RIGHTS). Native counterpart of the reference's Python
// `_exchange_ipc_fds` (moonep/buffer.py:113-179): every rank binds `<dir>/rank_<i>`,
// (the caller barriers,) sends its fd to every rank and receives one fd per sender.
// The three phases are separate calls so the collective barriers stay in Python.
#include "launch.h"
#include <errno.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

namespace {
struct Endpoint { int sock; int rank; int world; char dir[96]; };

int make_addr(sockaddr_un* a, const char* dir, int rank) {
  memset(a, 0, sizeof *a);
  a->sun_family = AF_UNIX;
  int n = snprintf(a->sun_path, sizeof a->sun_path, "%s/rank_%d", dir, rank);
  return (n > 0 && (size_t)n < sizeof a->sun_path) ? 0 : -1;
}
}  // namespace

extern "C" {

int mep_ipc_open(const char* dir, int rank, int world, void** ep_out) {
  MEP_REQUIRE(strlen(dir) < 80, "ipc: socket directory path too long: %s", dir);
  Endpoint* ep = new Endpoint{-1, rank, world, {0}};
  snprintf(ep->dir, sizeof ep->dir, "%s", dir);
  ep->sock = socket(AF_UNIX, SOCK_DGRAM, 0);
  if (ep->sock < 0) { delete ep; return mep::set_error("ipc: socket(): %s", strerror(errno)); }
  sockaddr_un a;
  if (make_addr(&a, dir, rank) || bind(ep->sock, (sockaddr*)&a, sizeof a) != 0) {
    int e = errno; close(ep->sock); delete ep;
    return mep::set_error("ipc: bind(%s/rank_%d): %s", dir, rank, strerror(e));
  }
  *ep_out = ep;
  return 0;
}

// Send `fd` to every rank in [0, world), tagging the message with the sender's rank.
int mep_ipc_send_all(void* epv, int fd) {
  Endpoint* ep = static_cast<Endpoint*>(epv);
  for (int dst = 0; dst < ep->world; ++dst) {
    sockaddr_un a; make_addr(&a, ep->dir, dst);
    int tag = ep->rank;
    iovec iov = {&tag, sizeof tag};
    char ctrl[CMSG_SPACE(sizeof(int))]; memset(ctrl, 0, sizeof ctrl);
    msghdr msg = {}; msg.msg_name = &a; msg.msg_namelen = sizeof a; msg.msg_iov = &iov; msg.msg_iovlen = 1;
    msg.msg_control = ctrl; msg.msg_controllen = sizeof ctrl;
    cmsghdr* cm = CMSG_FIRSTHDR(&msg);
    cm->cmsg_level = SOL_SOCKET; cm->cmsg_type = SCM_RIGHTS; cm->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(cm), &fd, sizeof fd);
    if (sendmsg(ep->sock, &msg, 0) < 0)
      return mep::set_error("ipc: sendmsg to rank %d: %s", dst, strerror(errno));
  }
  return 0;
}

// Receive one fd from every rank; fds_out[sender] = received descriptor. On timeout or a
// malformed message every descriptor received so far is closed and an error is returned.
int mep_ipc_recv_all(void* epv, int* fds_out, int timeout_ms) {
  Endpoint* ep = static_cast<Endpoint*>(epv);
  for (int i = 0; i < ep->world; ++i) fds_out[i] = -1;
  int got = 0;
  const char* why = nullptr; char whybuf[160];
  while (got < ep->world) {
    pollfd pfd = {ep->sock, POLLIN, 0};
    int pr = poll(&pfd, 1, timeout_ms);
    if (pr == 0) { snprintf(whybuf, sizeof whybuf, "timed out after %d ms with %d of %d descriptors", timeout_ms, got, ep->world); why = whybuf; break; }
    if (pr < 0) { if (errno == EINTR) continue; snprintf(whybuf, sizeof whybuf, "poll: %s", strerror(errno)); why = whybuf; break; }
    int tag = -1; iovec iov = {&tag, sizeof tag};
    char ctrl[CMSG_SPACE(sizeof(int))];
    msghdr msg = {}; msg.msg_iov = &iov; msg.msg_iovlen = 1; msg.msg_control = ctrl; msg.msg_controllen = sizeof ctrl;
    ssize_t n = recvmsg(ep->sock, &msg, 0);
    cmsghdr* cm = n == (ssize_t)sizeof tag ? CMSG_FIRSTHDR(&msg) : nullptr;
    int fd = -1;
    if (cm && cm->cmsg_level == SOL_SOCKET && cm->cmsg_type == SCM_RIGHTS) memcpy(&fd, CMSG_DATA(cm), sizeof fd);
    if (fd < 0 || tag < 0 || tag >= ep->world || fds_out[tag] >= 0) {
      if (fd >= 0) close(fd);
      snprintf(whybuf, sizeof whybuf, "malformed or duplicate message (sender tag %d)", tag); why = whybuf; break;
    }
    fds_out[tag] = fd; ++got;
  }
  if (why) {
    for (int i = 0; i < ep->world; ++i) if (fds_out[i] >= 0) { close(fds_out[i]); fds_out[i] = -1; }
    return mep::set_error("ipc: %s", why);
  }
  return 0;
}

int mep_ipc_close(void* epv) {
  Endpoint* ep = static_cast<Endpoint*>(epv);
  if (!ep) return 0;
  if (ep->sock >= 0) close(ep->sock);
  sockaddr_un a;
  if (make_addr(&a, ep->dir, ep->rank) == 0) unlink(a.sun_path);
  delete ep;
  return 0;
}

int mep_close_fd(int fd) { return fd >= 0 ? close(fd) : 0; }

}  // extern "C"
