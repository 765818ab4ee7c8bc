// Symmetric buckets for the fused ZeRO-1 path without any framework: one allocation per rank made with the
// CUDA virtual-memory API, mapped into every rank's process (peer mappings over NVLink) and, where the
// fabric supports it, bound to one NVSwitch multicast object.  The pointers go to nbo_zero1_attach_symmetric.
//
// The ranks are processes of one node.  What has to travel between them are file descriptors (the
// shareable handles of the allocations and of the multicast object), which cannot go through a byte
// channel; so the caller ships one 16-byte token (made by rank 0, like the NCCL unique id) and the library
// does the rest itself over abstract-namespace unix datagram sockets named after the token, passing the
// descriptors with SCM_RIGHTS.  Every wait has a time limit; on expiry the call fails with
// NBO_ERR_TIMEOUT and everything made so far is released.
//
// Order of the collective set-up (the multicast part follows the driver's rules: every device is added
// before any memory is bound):
//   1. every rank: cuMemCreate (shareable), map it locally, send its descriptor to every other rank
//   2. every rank: import the other ranks' descriptors, map them, allow this device to access them
//   3. rank 0: cuMulticastCreate, send its descriptor; every rank: cuMulticastAddDevice;   barrier
//   4. every rank: cuMulticastBindMem of its own allocation, map the multicast object;     barrier
// nbo_symm_free undoes it in reverse (unbind before anything is unmapped or released).
#include <cuda.h>
#include <errno.h>
#include <fcntl.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <chrono>
#include <random>
#include <string>
#include <vector>

#include "internal.h"

namespace nbo {

// The driver entry points, fetched through the runtime so that the library does not link libcuda.
struct DriverApi {
    bool ok = false;
    std::string why;
#define NBO_DRV(name) decltype(&name) name##_ = nullptr;
    NBO_DRV(cuMemCreate)
    NBO_DRV(cuMemRelease)
    NBO_DRV(cuMemExportToShareableHandle)
    NBO_DRV(cuMemImportFromShareableHandle)
    NBO_DRV(cuMemAddressReserve)
    NBO_DRV(cuMemAddressFree)
    NBO_DRV(cuMemMap)
    NBO_DRV(cuMemUnmap)
    NBO_DRV(cuMemSetAccess)
    NBO_DRV(cuMemGetAllocationGranularity)
    NBO_DRV(cuMulticastCreate)
    NBO_DRV(cuMulticastAddDevice)
    NBO_DRV(cuMulticastBindMem)
    NBO_DRV(cuMulticastUnbind)
    NBO_DRV(cuMulticastGetGranularity)
    NBO_DRV(cuDeviceGet)
    NBO_DRV(cuDeviceGetAttribute)
    NBO_DRV(cuGetErrorString)
#undef NBO_DRV
};

static DriverApi *driver_api()
{
    static DriverApi api;
    if (api.ok || !api.why.empty()) return &api;
    auto get = [&](const char *name, void **fn) {
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q);
        if ((e != cudaSuccess || q != cudaDriverEntryPointSuccess || !*fn) && api.why.empty())
            api.why = std::string("nabla-optim-b200: the CUDA driver does not provide ") + name;
    };
#define NBO_DRV(name) get(#name, (void **)&api.name##_);
    NBO_DRV(cuMemCreate)
    NBO_DRV(cuMemRelease)
    NBO_DRV(cuMemExportToShareableHandle)
    NBO_DRV(cuMemImportFromShareableHandle)
    NBO_DRV(cuMemAddressReserve)
    NBO_DRV(cuMemAddressFree)
    NBO_DRV(cuMemMap)
    NBO_DRV(cuMemUnmap)
    NBO_DRV(cuMemSetAccess)
    NBO_DRV(cuMemGetAllocationGranularity)
    NBO_DRV(cuMulticastCreate)
    NBO_DRV(cuMulticastAddDevice)
    NBO_DRV(cuMulticastBindMem)
    NBO_DRV(cuMulticastUnbind)
    NBO_DRV(cuMulticastGetGranularity)
    NBO_DRV(cuDeviceGet)
    NBO_DRV(cuDeviceGetAttribute)
    NBO_DRV(cuGetErrorString)
#undef NBO_DRV
    api.ok = api.why.empty();
    return &api;
}

using SymmClock = std::chrono::steady_clock;

// One message of the set-up protocol; a descriptor may ride along as ancillary data.
struct SymmMsg {
    int32_t type;  // 1 allocation descriptor, 2 multicast descriptor, 3 arrived at barrier, 4 barrier released
    int32_t rank;
    int32_t phase;
    int32_t pad;
};

}  // namespace nbo

struct nbo_symm {
    int device = 0, rank = 0, world = 1;
    size_t bytes = 0;      // as asked
    size_t mapped = 0;     // rounded up to the granularity
    std::string err;
    std::string name_prefix;
    int sock = -1;
    std::vector<nbo::SymmMsg> inbox;  // messages that arrived before they were waited for
    std::vector<int> inbox_fd;
    CUmemGenericAllocationHandle local_h = 0;
    std::vector<CUmemGenericAllocationHandle> peer_h;  // [world]; [rank] unused
    std::vector<CUdeviceptr> va;                       // [world]; va[rank] is the local mapping
    std::vector<bool> va_mapped;
    CUmemGenericAllocationHandle mc_h = 0;
    bool mc_added = false, mc_bound = false;
    CUdeviceptr mc_va = 0;
    bool mc_mapped = false;
    double timeout_s = 60.0;
};

namespace nbo {

static int32_t symm_fail(nbo_symm *s, int32_t code, const std::string &msg)
{
    if (s) s->err = msg;
    return fail(nullptr, code, msg);
}

static int32_t symm_drv(nbo_symm *s, CUresult r, const char *what)
{
    if (r == CUDA_SUCCESS) return NBO_OK;
    const char *txt = nullptr;
    driver_api()->cuGetErrorString_(r, &txt);
    int32_t code = r == CUDA_ERROR_OUT_OF_MEMORY ? NBO_ERR_NOMEM : NBO_ERR_CUDA;
    return symm_fail(s, code, std::string("CUDA driver error: ") + (txt ? txt : "?") + " in " + what);
}

#define NBO_DRVCALL(s, call)                                   \
    do {                                                       \
        int32_t rc__ = nbo::symm_drv((s), (call), #call);      \
        if (rc__ != NBO_OK) return rc__;                       \
    } while (0)

static sockaddr_un symm_addr(const std::string &prefix, int rank, socklen_t *len)
{
    sockaddr_un a;
    memset(&a, 0, sizeof(a));
    a.sun_family = AF_UNIX;
    std::string n = prefix + "-" + std::to_string(rank);
    // abstract namespace: sun_path[0] == 0, no file system entry, gone when the socket closes
    memcpy(a.sun_path + 1, n.data(), n.size());
    *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n.size());
    return a;
}

static int32_t symm_send(nbo_symm *s, int to, const SymmMsg &m, int fd, SymmClock::time_point deadline)
{
    socklen_t alen;
    sockaddr_un addr = symm_addr(s->name_prefix, to, &alen);
    msghdr mh;
    memset(&mh, 0, sizeof(mh));
    iovec iov{(void *)&m, sizeof(m)};
    mh.msg_name = &addr;
    mh.msg_namelen = alen;
    mh.msg_iov = &iov;
    mh.msg_iovlen = 1;
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
    if (fd >= 0) {
        memset(ctrl, 0, sizeof(ctrl));
        mh.msg_control = ctrl;
        mh.msg_controllen = sizeof(ctrl);
        cmsghdr *c = CMSG_FIRSTHDR(&mh);
        c->cmsg_level = SOL_SOCKET;
        c->cmsg_type = SCM_RIGHTS;
        c->cmsg_len = CMSG_LEN(sizeof(int));
        memcpy(CMSG_DATA(c), &fd, sizeof(int));
    }
    for (;;) {
        if (sendmsg(s->sock, &mh, 0) >= 0) return NBO_OK;
        // the peer has not bound its socket yet (or its queue is full): try again until the limit
        if (errno != ECONNREFUSED && errno != ENOENT && errno != EAGAIN && errno != ENOBUFS && errno != EINTR)
            return symm_fail(s, NBO_ERR_STATE, std::string("nabla-optim-b200: sendmsg to rank ") + std::to_string(to) +
                                                   " failed: " + strerror(errno));
        if (SymmClock::now() > deadline)
            return symm_fail(s, NBO_ERR_TIMEOUT, "nabla-optim-b200: timed out reaching rank " + std::to_string(to) +
                                                     " while setting up symmetric memory (did every rank call in?)");
        usleep(2000);
    }
}

// Waits for the message (type, phase) from `from` (-1 = any rank); other messages are kept for later.
static int32_t symm_recv(nbo_symm *s, int type, int phase, int from, int *from_out, int *fd_out,
                         SymmClock::time_point deadline)
{
    for (;;) {
        for (size_t i = 0; i < s->inbox.size(); ++i) {
            const SymmMsg &m = s->inbox[i];
            if (m.type == type && m.phase == phase && (from < 0 || m.rank == from)) {
                if (from_out) *from_out = m.rank;
                if (fd_out) *fd_out = s->inbox_fd[i];
                else if (s->inbox_fd[i] >= 0) close(s->inbox_fd[i]);
                s->inbox.erase(s->inbox.begin() + i);
                s->inbox_fd.erase(s->inbox_fd.begin() + i);
                return NBO_OK;
            }
        }
        auto now = SymmClock::now();
        if (now > deadline)
            return symm_fail(s, NBO_ERR_TIMEOUT, "nabla-optim-b200: timed out waiting for the other ranks while setting up "
                                                 "symmetric memory");
        int ms = (int)std::chrono::duration_cast<std::chrono::milliseconds>(deadline - now).count();
        pollfd p{s->sock, POLLIN, 0};
        int pr = poll(&p, 1, ms < 1 ? 1 : (ms > 200 ? 200 : ms));
        if (pr < 0 && errno != EINTR)
            return symm_fail(s, NBO_ERR_STATE, std::string("nabla-optim-b200: poll failed: ") + strerror(errno));
        if (pr <= 0) continue;
        SymmMsg m;
        msghdr mh;
        memset(&mh, 0, sizeof(mh));
        iovec iov{&m, sizeof(m)};
        mh.msg_iov = &iov;
        mh.msg_iovlen = 1;
        alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
        mh.msg_control = ctrl;
        mh.msg_controllen = sizeof(ctrl);
        ssize_t n = recvmsg(s->sock, &mh, MSG_DONTWAIT);
        if (n < 0) {
            if (errno == EAGAIN || errno == EINTR) continue;
            return symm_fail(s, NBO_ERR_STATE, std::string("nabla-optim-b200: recvmsg failed: ") + strerror(errno));
        }
        if (n != (ssize_t)sizeof(m)) continue;
        int fd = -1;
        for (cmsghdr *c = CMSG_FIRSTHDR(&mh); c; c = CMSG_NXTHDR(&mh, c))
            if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) memcpy(&fd, CMSG_DATA(c), sizeof(int));
        s->inbox.push_back(m);
        s->inbox_fd.push_back(fd);
    }
}

// All ranks arrive, rank 0 releases.
static int32_t symm_barrier(nbo_symm *s, int phase, SymmClock::time_point deadline)
{
    if (s->world == 1) return NBO_OK;
    int32_t rc;
    if (s->rank == 0) {
        for (int i = 1; i < s->world; ++i)
            if ((rc = symm_recv(s, 3, phase, -1, nullptr, nullptr, deadline)) != NBO_OK) return rc;
        for (int r = 1; r < s->world; ++r)
            if ((rc = symm_send(s, r, SymmMsg{4, 0, phase, 0}, -1, deadline)) != NBO_OK) return rc;
        return NBO_OK;
    }
    if ((rc = symm_send(s, 0, SymmMsg{3, s->rank, phase, 0}, -1, deadline)) != NBO_OK) return rc;
    return symm_recv(s, 4, phase, 0, nullptr, nullptr, deadline);
}

static void symm_release(nbo_symm *s)
{
    DriverApi *d = driver_api();
    if (!d->ok) return;
    cudaDeviceSynchronize();
    CUdevice dev = 0;
    d->cuDeviceGet_(&dev, s->device);
    // the multicast binding goes first: nothing it refers to may disappear underneath it
    if (s->mc_mapped) { d->cuMemUnmap_(s->mc_va, s->mapped); s->mc_mapped = false; }
    if (s->mc_va) { d->cuMemAddressFree_(s->mc_va, s->mapped); s->mc_va = 0; }
    if (s->mc_bound) { d->cuMulticastUnbind_(s->mc_h, dev, 0, s->mapped); s->mc_bound = false; }
    if (s->mc_h) { d->cuMemRelease_(s->mc_h); s->mc_h = 0; }
    for (int r = 0; r < (int)s->va.size(); ++r) {
        if (s->va_mapped[r]) { d->cuMemUnmap_(s->va[r], s->mapped); s->va_mapped[r] = false; }
        if (s->va[r]) { d->cuMemAddressFree_(s->va[r], s->mapped); s->va[r] = 0; }
        if (r != s->rank && r < (int)s->peer_h.size() && s->peer_h[r]) { d->cuMemRelease_(s->peer_h[r]); s->peer_h[r] = 0; }
    }
    if (s->local_h) { d->cuMemRelease_(s->local_h); s->local_h = 0; }
    for (int fd : s->inbox_fd)
        if (fd >= 0) close(fd);
    s->inbox.clear();
    s->inbox_fd.clear();
    if (s->sock >= 0) { close(s->sock); s->sock = -1; }
}

static int32_t symm_setup(nbo_symm *s, int want_multicast)
{
    DriverApi *d = driver_api();
    const SymmClock::time_point deadline =
        SymmClock::now() + std::chrono::duration_cast<SymmClock::duration>(std::chrono::duration<double>(s->timeout_s));
    CUdevice dev;
    NBO_DRVCALL(s, d->cuDeviceGet_(&dev, s->device));

    CUmemAllocationProp prop;
    memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = s->device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t gran = 0;
    NBO_DRVCALL(s, d->cuMemGetAllocationGranularity_(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));

    int mc_supported = 0;
    if (want_multicast && s->world > 1)
        d->cuDeviceGetAttribute_(&mc_supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev);
    CUmulticastObjectProp mcprop;
    memset(&mcprop, 0, sizeof(mcprop));
    if (mc_supported) {
        mcprop.numDevices = (unsigned)s->world;
        mcprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        mcprop.size = s->bytes;
        size_t mgran = 0;
        if (d->cuMulticastGetGranularity_(&mgran, &mcprop, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mgran > gran)
            gran = mgran;
    }
    s->mapped = (s->bytes + gran - 1) / gran * gran;
    mcprop.size = s->mapped;

    s->peer_h.assign(s->world, 0);
    s->va.assign(s->world, 0);
    s->va_mapped.assign(s->world, false);
    CUmemAccessDesc access;
    memset(&access, 0, sizeof(access));
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = s->device;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;

    // 1. this rank's allocation
    NBO_DRVCALL(s, d->cuMemCreate_(&s->local_h, s->mapped, &prop, 0));
    NBO_DRVCALL(s, d->cuMemAddressReserve_(&s->va[s->rank], s->mapped, gran, 0, 0));
    NBO_DRVCALL(s, d->cuMemMap_(s->va[s->rank], s->mapped, 0, s->local_h, 0));
    s->va_mapped[s->rank] = true;
    NBO_DRVCALL(s, d->cuMemSetAccess_(s->va[s->rank], s->mapped, &access, 1));
    if (s->world == 1) return NBO_OK;

    int my_fd = -1;
    NBO_DRVCALL(s, d->cuMemExportToShareableHandle_(&my_fd, s->local_h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
    int32_t rc = NBO_OK;
    for (int r = 0; r < s->world && rc == NBO_OK; ++r)
        if (r != s->rank) rc = symm_send(s, r, SymmMsg{1, s->rank, 0, 0}, my_fd, deadline);
    close(my_fd);
    if (rc != NBO_OK) return rc;

    // 2. the other ranks' allocations
    for (int i = 1; i < s->world; ++i) {
        int from = -1, fd = -1;
        if ((rc = symm_recv(s, 1, 0, -1, &from, &fd, deadline)) != NBO_OK) return rc;
        if (from < 0 || from >= s->world || from == s->rank || fd < 0 || s->peer_h[from]) {
            if (fd >= 0) close(fd);
            return symm_fail(s, NBO_ERR_STATE, "nabla-optim-b200: unexpected descriptor message while setting up symmetric memory");
        }
        CUresult r = d->cuMemImportFromShareableHandle_(&s->peer_h[from], (void *)(uintptr_t)fd,
                                                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
        close(fd);
        NBO_DRVCALL(s, r);
        NBO_DRVCALL(s, d->cuMemAddressReserve_(&s->va[from], s->mapped, gran, 0, 0));
        NBO_DRVCALL(s, d->cuMemMap_(s->va[from], s->mapped, 0, s->peer_h[from], 0));
        s->va_mapped[from] = true;
        NBO_DRVCALL(s, d->cuMemSetAccess_(s->va[from], s->mapped, &access, 1));
    }
    if ((rc = symm_barrier(s, 1, deadline)) != NBO_OK) return rc;  // every rank holds every mapping
    if (!mc_supported) return NBO_OK;

    // 3. the multicast object: created by rank 0, every device added before anything is bound
    if (s->rank == 0) {
        NBO_DRVCALL(s, d->cuMulticastCreate_(&s->mc_h, &mcprop));
        int mc_fd = -1;
        NBO_DRVCALL(s, d->cuMemExportToShareableHandle_(&mc_fd, s->mc_h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
        for (int r = 1; r < s->world && rc == NBO_OK; ++r) rc = symm_send(s, r, SymmMsg{2, 0, 0, 0}, mc_fd, deadline);
        close(mc_fd);
        if (rc != NBO_OK) return rc;
    } else {
        int fd = -1;
        if ((rc = symm_recv(s, 2, 0, 0, nullptr, &fd, deadline)) != NBO_OK) return rc;
        if (fd < 0) return symm_fail(s, NBO_ERR_STATE, "nabla-optim-b200: the multicast descriptor did not arrive");
        CUresult r = d->cuMemImportFromShareableHandle_(&s->mc_h, (void *)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
        close(fd);
        NBO_DRVCALL(s, r);
    }
    NBO_DRVCALL(s, d->cuMulticastAddDevice_(s->mc_h, dev));
    s->mc_added = true;
    if ((rc = symm_barrier(s, 2, deadline)) != NBO_OK) return rc;

    // 4. bind this rank's memory and map the object
    NBO_DRVCALL(s, d->cuMulticastBindMem_(s->mc_h, 0, s->local_h, 0, s->mapped, 0));
    s->mc_bound = true;
    NBO_DRVCALL(s, d->cuMemAddressReserve_(&s->mc_va, s->mapped, gran, 0, 0));
    NBO_DRVCALL(s, d->cuMemMap_(s->mc_va, s->mapped, 0, s->mc_h, 0));
    s->mc_mapped = true;
    NBO_DRVCALL(s, d->cuMemSetAccess_(s->mc_va, s->mapped, &access, 1));
    return symm_barrier(s, 3, deadline);  // every rank is bound before anyone uses the multicast address
}

}  // namespace nbo

using namespace nbo;

extern "C" {

int32_t nbo_symm_token(uint8_t token_out[16])
{
    if (!token_out) return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: null token buffer");
    std::random_device rd;
    for (int i = 0; i < 16; i += 4) {
        uint32_t v = rd() ^ (uint32_t)getpid() ^ (uint32_t)SymmClock::now().time_since_epoch().count();
        memcpy(token_out + i, &v, 4);
    }
    return NBO_OK;
}

int32_t nbo_symm_alloc(int32_t device, int32_t rank, int32_t world, uint64_t bytes, const uint8_t token[16],
                       int32_t tag, int32_t want_multicast, double timeout_s, nbo_symm **out)
{
    if (!out) return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: nbo_symm_alloc: null out pointer");
    *out = nullptr;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
        return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: nbo_symm_alloc: rank/world out of range");
    if (bytes == 0) return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: nbo_symm_alloc: zero size");
    if (world > 1 && !token) return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: nbo_symm_alloc: world > 1 needs the token");
    if (!(timeout_s > 0.0)) timeout_s = 60.0;
    DeviceGuard guard(device);
    cudaError_t ce = cudaFree(nullptr);  // makes sure the device's primary context exists and is current
    if (ce != cudaSuccess) return fail_cuda(nullptr, ce, "cudaFree(0)");
    DriverApi *d = driver_api();
    if (!d->ok) return fail(nullptr, NBO_ERR_CUDA, d->why);

    nbo_symm *s = new (std::nothrow) nbo_symm();
    if (!s) return fail(nullptr, NBO_ERR_NOMEM, "nabla-optim-b200: out of host memory");
    s->device = device; s->rank = rank; s->world = world; s->bytes = bytes; s->timeout_s = timeout_s;
    if (world > 1) {
        char hex[33];
        for (int i = 0; i < 16; ++i) snprintf(hex + 2 * i, 3, "%02x", token[i]);
        s->name_prefix = std::string("nbo-symm-") + hex + "-" + std::to_string(tag);
        s->sock = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
        socklen_t alen;
        sockaddr_un addr = symm_addr(s->name_prefix, rank, &alen);
        if (s->sock < 0 || bind(s->sock, (sockaddr *)&addr, alen) != 0) {
            std::string m = std::string("nabla-optim-b200: cannot open the set-up socket: ") + strerror(errno);
            symm_release(s);
            delete s;
            return fail(nullptr, NBO_ERR_STATE, m);
        }
    }
    int32_t rc = symm_setup(s, want_multicast);
    if (rc != NBO_OK) {
        std::string m = s->err;
        symm_release(s);
        delete s;
        return fail(nullptr, rc, m);
    }
    if (s->sock >= 0) { close(s->sock); s->sock = -1; }  // the set-up is over; nothing else uses the sockets
    *out = s;
    return NBO_OK;
}

int32_t nbo_symm_pointers(const nbo_symm *s, void **local, void **peers, void **multicast)
{
    if (!s) return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: null symmetric allocation");
    if (local) *local = (void *)s->va[s->rank];
    if (peers)
        for (int r = 0; r < s->world; ++r) peers[r] = (void *)s->va[r];
    if (multicast) *multicast = s->mc_mapped ? (void *)s->mc_va : nullptr;
    return NBO_OK;
}

int32_t nbo_symm_free(nbo_symm *s)
{
    if (!s) return NBO_OK;
    DeviceGuard guard(s->device);
    symm_release(s);
    delete s;
    return NBO_OK;
}

}  // extern "C"
