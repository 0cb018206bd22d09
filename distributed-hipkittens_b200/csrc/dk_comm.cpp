// Host bootstrap between the ranks of one node, without MPI.
//
// Stands in for what the reference gets from iris::mpi::initialize / MPI under iris
// (distributed-kernels/iris_py.cpp:55-57,149-154; distributed-kernels/CMakeLists.txt:95,122):
// rank discovery, a host barrier, and the exchange of the handles that let every rank map every
// other rank's heap. Here: rank and world come from the environment, ranks meet on an abstract
// Unix-domain socket (star around rank 0), file descriptors travel with SCM_RIGHTS.
// Pure host code with no CUDA in it, so it is testable on a machine without a GPU.
//
// Who may join: the socket name is predictable, and whoever joins receives the descriptors of every
// rank's heap. Rank 0 therefore accepts a connection only from a process of its own user
// (SO_PEERCRED) whose hello carries the job's token (DK_JOB_TOKEN in the environment of all ranks; 0
// when unset); connections are accepted at once and their hello read when it arrives, so a silent
// connection holds up nobody; anything else is dropped without giving up the job.
#include <errno.h>
#include <poll.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/dk_b200.h"

namespace dk {
void set_last_error(const std::string& s);
void log_msg(int level, const std::string& s);
}

struct dk_comm {
    int rank = 0;
    int world = 1;
    int timeout_ms = 60000;
    int listen_fd = -1;
    std::vector<int> peers;  // rank 0: socket to each rank (peers[0] unused); others: peers[0] = socket to rank 0
};

namespace {

int64_t now_ms() {
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return static_cast<int64_t>(ts.tv_sec) * 1000 + ts.tv_nsec / 1000000;
}

int fail(const std::string& what) {
    dk::set_last_error("bootstrap: " + what + (errno ? std::string(": ") + strerror(errno) : ""));
    return DK_ERR_BOOTSTRAP;
}

bool wait_fd(int fd, short events, int timeout_ms) {
    pollfd p{fd, events, 0};
    for (;;) {
        int r = poll(&p, 1, timeout_ms);
        if (r > 0) return (p.revents & events) != 0;
        if (r == 0) {
            errno = ETIMEDOUT;
            return false;
        }
        if (errno != EINTR) return false;
    }
}

bool send_all(int fd, const void* buf, size_t n) {
    const char* p = static_cast<const char*>(buf);
    while (n > 0) {
        ssize_t w = send(fd, p, n, MSG_NOSIGNAL);
        if (w < 0) {
            if (errno == EINTR) continue;
            return false;
        }
        p += w;
        n -= static_cast<size_t>(w);
    }
    return true;
}

bool recv_all(int fd, void* buf, size_t n, int timeout_ms) {
    char* p = static_cast<char*>(buf);
    while (n > 0) {
        if (!wait_fd(fd, POLLIN, timeout_ms)) return false;
        ssize_t r = recv(fd, p, n, 0);
        if (r == 0) {
            errno = ECONNRESET;  // peer closed: it exited or was killed
            return false;
        }
        if (r < 0) {
            if (errno == EINTR) continue;
            return false;
        }
        p += r;
        n -= static_cast<size_t>(r);
    }
    return true;
}

bool send_fd(int sock, int fd) {
    char byte = 'F';
    iovec io{&byte, 1};
    char ctrl[CMSG_SPACE(sizeof(int))];
    memset(ctrl, 0, sizeof(ctrl));
    msghdr msg{};
    msg.msg_iov = &io;
    msg.msg_iovlen = 1;
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(c), &fd, sizeof(int));
    for (;;) {
        ssize_t w = sendmsg(sock, &msg, MSG_NOSIGNAL);
        if (w == 1) return true;
        if (w < 0 && errno == EINTR) continue;
        return false;
    }
}

bool recv_fd(int sock, int* fd, int timeout_ms) {
    if (!wait_fd(sock, POLLIN, timeout_ms)) return false;
    char byte = 0;
    iovec io{&byte, 1};
    char ctrl[CMSG_SPACE(sizeof(int))];
    memset(ctrl, 0, sizeof(ctrl));
    msghdr msg{};
    msg.msg_iov = &io;
    msg.msg_iovlen = 1;
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    for (;;) {
        ssize_t r = recvmsg(sock, &msg, 0);
        if (r == 1) break;
        if (r == 0) {
            errno = ECONNRESET;
            return false;
        }
        if (r < 0 && errno == EINTR) continue;
        return false;
    }
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    if (c == nullptr || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) {
        errno = EPROTO;
        return false;
    }
    memcpy(fd, CMSG_DATA(c), sizeof(int));
    return true;
}

// Abstract-namespace address: no file is left behind when a rank dies.
socklen_t make_addr(const std::string& name, sockaddr_un* a) {
    memset(a, 0, sizeof(*a));
    a->sun_family = AF_UNIX;
    std::string n = "dk_b200." + name;
    if (n.size() > sizeof(a->sun_path) - 2) n.resize(sizeof(a->sun_path) - 2);
    a->sun_path[0] = '\0';
    memcpy(a->sun_path + 1, n.data(), n.size());
    return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n.size());
}

std::atomic<int> g_comm_seq{0};

struct Hello {
    int32_t rank;
    uint32_t magic;
    uint64_t token;
};
constexpr uint32_t HELLO_MAGIC = 0x646b3230u;

// FNV-1a of DK_JOB_TOKEN (0 when unset): ranks of one job share it through their environment.
uint64_t job_token() {
    const char* t = getenv("DK_JOB_TOKEN");
    if (t == nullptr || *t == '\0') return 0;
    uint64_t h = 1469598103934665603ull;
    for (; *t; ++t) h = (h ^ static_cast<unsigned char>(*t)) * 1099511628211ull;
    return h ? h : 1;
}

bool same_user(int s) {
    ucred cr{};
    socklen_t len = sizeof(cr);
    if (getsockopt(s, SOL_SOCKET, SO_PEERCRED, &cr, &len) != 0) return false;
    return cr.uid == geteuid();
}

// Empty when neither DK_JOB_ID nor MASTER_PORT names the job (two jobs of one host would otherwise
// meet on the same default name).
std::string default_rendezvous() {
    std::string base;
    if (const char* e = getenv("DK_JOB_ID")) base = e;
    else if (const char* p = getenv("MASTER_PORT")) base = std::string("port") + p;
    else return std::string();
    // heaps are created in the same order on every rank, so a per-process counter pairs them up
    return base + "." + std::to_string(g_comm_seq.fetch_add(1));
}

int env_int(const char* a, const char* b, int dflt) {
    const char* v = getenv(a);
    if (v == nullptr && b != nullptr) v = getenv(b);
    if (v == nullptr || *v == '\0') return dflt;
    return atoi(v);
}

}  // namespace

extern "C" {

int dk_bootstrap_env(int* rank, int* world, int* local_rank) {
    if (rank == nullptr || world == nullptr || local_rank == nullptr) return DK_ERR_ARG;
    *rank = env_int("RANK", "OMPI_COMM_WORLD_RANK", 0);
    *world = env_int("WORLD_SIZE", "OMPI_COMM_WORLD_SIZE", 1);
    *local_rank = env_int("LOCAL_RANK", "OMPI_COMM_WORLD_LOCAL_RANK", *rank);
    if (*world < 1 || *rank < 0 || *rank >= *world) {
        dk::set_last_error("bootstrap: inconsistent RANK/WORLD_SIZE in the environment");
        return DK_ERR_BOOTSTRAP;
    }
    return DK_OK;
}

int dk_comm_create(int rank, int world, const char* rendezvous, int timeout_ms, dk_comm** out) {
    if (out == nullptr || world < 1 || world > DK_MAX_RANKS || rank < 0 || rank >= world) {
        dk::set_last_error("argument error: dk_comm_create rank/world");
        return DK_ERR_ARG;
    }
    errno = 0;
    dk_comm* c = new dk_comm;
    c->rank = rank;
    c->world = world;
    c->timeout_ms = timeout_ms > 0 ? timeout_ms : 60000;
    *out = c;
    if (world == 1) return DK_OK;

    const std::string name = (rendezvous && *rendezvous) ? rendezvous : default_rendezvous();
    if (name.empty()) {
        errno = 0;
        int rc = fail("no rendezvous name: pass one, or set DK_JOB_ID (or MASTER_PORT, as torchrun does) in the "
                      "environment of every rank");
        delete c; *out = nullptr;
        return rc;
    }
    const uint64_t token = job_token();
    sockaddr_un addr;
    const socklen_t alen = make_addr(name, &addr);
    const int64_t deadline = now_ms() + c->timeout_ms;

    if (rank == 0) {
        c->peers.assign(world, -1);
        c->listen_fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
        if (c->listen_fd < 0) { delete c; *out = nullptr; return fail("socket"); }
        if (bind(c->listen_fd, reinterpret_cast<sockaddr*>(&addr), alen) != 0 ||
            listen(c->listen_fd, world) != 0) {
            int rc = fail("bind/listen on rendezvous '" + name + "'");
            close(c->listen_fd); delete c; *out = nullptr;
            return rc;
        }
        // Connections are accepted at once and their hello is read when it arrives, so a connection
        // that says nothing holds up nobody. A stranger (other user), a wrong token or magic, a rank
        // out of range or already here: dropped, and the loop goes on waiting for the real ranks.
        std::vector<int> pending;
        auto drop_pending = [&]() {
            for (int fd : pending) close(fd);
            pending.clear();
        };
        for (int got = 0; got < world - 1;) {
            const int left = static_cast<int>(deadline - now_ms());
            std::vector<pollfd> pf;
            pf.push_back({c->listen_fd, POLLIN, 0});
            for (int fd : pending) pf.push_back({fd, POLLIN, 0});
            const int pr = left > 0 ? poll(pf.data(), pf.size(), left) : 0;
            if (pr < 0 && errno == EINTR) continue;
            if (pr <= 0) {
                errno = ETIMEDOUT;
                int rc = fail("timed out waiting for " + std::to_string(world - 1 - got) +
                              " rank(s) at rendezvous '" + name + "'");
                drop_pending();
                dk_comm_destroy(c); *out = nullptr;
                return rc;
            }
            std::vector<int> still;
            for (size_t i = 1; i < pf.size(); ++i) {
                const int s = pf[i].fd;
                if ((pf[i].revents & (POLLIN | POLLHUP | POLLERR)) == 0) {
                    still.push_back(s);
                    continue;
                }
                Hello h{-1, 0, 0};
                if (!recv_all(s, &h, sizeof(h), 1000) || h.magic != HELLO_MAGIC || h.token != token || h.rank <= 0 ||
                    h.rank >= world || c->peers[h.rank] != -1) {
                    close(s);
                    dk::log_msg(2, "rendezvous '" + name + "': a connection without a valid hello was dropped");
                    continue;
                }
                c->peers[h.rank] = s;
                ++got;
                dk::log_msg(2, "rendezvous '" + name + "': rank " + std::to_string(h.rank) + " joined");
            }
            pending.swap(still);
            if (pf[0].revents & POLLIN) {
                const int s = accept4(c->listen_fd, nullptr, nullptr, SOCK_CLOEXEC);
                if (s >= 0) {
                    if (same_user(s)) pending.push_back(s);
                    else close(s);
                }
            }
        }
        drop_pending();
    } else {
        c->peers.assign(1, -1);
        for (;;) {
            int s = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
            if (s < 0) { delete c; *out = nullptr; return fail("socket"); }
            if (connect(s, reinterpret_cast<sockaddr*>(&addr), alen) == 0) {
                c->peers[0] = s;
                break;
            }
            close(s);
            if (now_ms() > deadline) {
                errno = ETIMEDOUT;
                int rc = fail("rank 0 never appeared at rendezvous '" + name + "'");
                delete c; *out = nullptr;
                return rc;
            }
            usleep(5000);
        }
        const Hello h{rank, HELLO_MAGIC, token};
        if (!send_all(c->peers[0], &h, sizeof(h))) {
            int rc = fail("hello to rank 0");
            dk_comm_destroy(c); *out = nullptr;
            return rc;
        }
    }
    int rc = dk_comm_barrier(c);
    if (rc != DK_OK) { dk_comm_destroy(c); *out = nullptr; }
    return rc;
}

int dk_comm_destroy(dk_comm* c) {
    if (c == nullptr) return DK_OK;
    for (int fd : c->peers)
        if (fd >= 0) close(fd);
    if (c->listen_fd >= 0) close(c->listen_fd);
    delete c;
    return DK_OK;
}

int dk_comm_barrier(dk_comm* c) {
    if (c == nullptr) return DK_ERR_ARG;
    if (c->world == 1) return DK_OK;
    errno = 0;
    char b = 'B';
    if (c->rank == 0) {
        for (int r = 1; r < c->world; ++r)
            if (!recv_all(c->peers[r], &b, 1, c->timeout_ms))
                return fail("barrier: rank " + std::to_string(r) + " did not arrive");
        for (int r = 1; r < c->world; ++r)
            if (!send_all(c->peers[r], &b, 1)) return fail("barrier: release to rank " + std::to_string(r));
    } else {
        if (!send_all(c->peers[0], &b, 1)) return fail("barrier: arrive");
        if (!recv_all(c->peers[0], &b, 1, c->timeout_ms)) return fail("barrier: no release from rank 0");
    }
    return DK_OK;
}

int dk_comm_allgather(dk_comm* c, const void* mine, size_t bytes, void* all_out) {
    if (c == nullptr || mine == nullptr || all_out == nullptr) return DK_ERR_ARG;
    char* all = static_cast<char*>(all_out);
    memcpy(all + static_cast<size_t>(c->rank) * bytes, mine, bytes);
    if (c->world == 1) return DK_OK;
    errno = 0;
    if (c->rank == 0) {
        for (int r = 1; r < c->world; ++r)
            if (!recv_all(c->peers[r], all + static_cast<size_t>(r) * bytes, bytes, c->timeout_ms))
                return fail("allgather: nothing from rank " + std::to_string(r));
        for (int r = 1; r < c->world; ++r)
            if (!send_all(c->peers[r], all, bytes * c->world)) return fail("allgather: send");
    } else {
        if (!send_all(c->peers[0], mine, bytes)) return fail("allgather: send");
        if (!recv_all(c->peers[0], all, bytes * c->world, c->timeout_ms))
            return fail("allgather: nothing from rank 0");
    }
    return DK_OK;
}

int dk_comm_allgather_fd(dk_comm* c, int my_fd, int* fds_out) {
    if (c == nullptr || fds_out == nullptr || my_fd < 0) return DK_ERR_ARG;
    errno = 0;
    for (int r = 0; r < c->world; ++r) fds_out[r] = -1;
    fds_out[c->rank] = dup(my_fd);
    if (fds_out[c->rank] < 0) return fail("dup");
    if (c->world == 1) return DK_OK;
    if (c->rank == 0) {
        for (int r = 1; r < c->world; ++r)
            if (!recv_fd(c->peers[r], &fds_out[r], c->timeout_ms))
                return fail("fd exchange: nothing from rank " + std::to_string(r));
        for (int r = 1; r < c->world; ++r)
            for (int k = 0; k < c->world; ++k) {
                if (k == r) continue;
                if (!send_fd(c->peers[r], fds_out[k])) return fail("fd exchange: send");
            }
    } else {
        if (!send_fd(c->peers[0], my_fd)) return fail("fd exchange: send");
        for (int k = 0; k < c->world; ++k) {
            if (k == c->rank) continue;
            if (!recv_fd(c->peers[0], &fds_out[k], c->timeout_ms))
                return fail("fd exchange: nothing from rank 0");
        }
    }
    return DK_OK;
}

}  // extern "C"
