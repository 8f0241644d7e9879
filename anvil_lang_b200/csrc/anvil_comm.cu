// anvil_comm.cu — the data-parallel collective inside the runtime: NCCL over NVLink / NVSwitch, no Python in the path.
//
// The reference has no multi-device code; the scheme (anvil_lang_b200/dp.py) needs exactly one collective, the sum of
// the gradient bucket over the ranks. NCCL is loaded with dlopen at the first use ("libnccl.so.2": the copy a host
// program has already loaded, e.g. torch's, or the system's), so libanvil_cuda.so has no link-time dependency on it
// and single-GPU processes never touch it.
//
//   rank 0:     anvil_rt_comm_unique_id(id)             128 bytes, handed to the other ranks by the host program
//   every rank: anvil_rt_comm_init(rt, rank, nranks, id, 128)
//   per step:   anvil_rt_allreduce(rt, off, count)      ncclAllReduce(sum, f32), in place on the arena, on the context's stream
//
// The call is stream-ordered like a kernel launch: the step's graphs before and after it need no host synchronisation.
// For run-to-run bit-identical sums at a given GPU count the algorithm, protocol and channel count are pinned before the
// communicator is made (NCCL_ALGO=Ring, NCCL_PROTO=Simple, NCCL_MIN_NCHANNELS = NCCL_MAX_NCHANNELS = 8) unless the
// environment already sets them: a ring with a fixed number of channels adds the ranks' contributions in a fixed order.
#include "anvil_cuda.h"

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>

namespace {

struct Nccl {
    void *lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommCount)(const ncclComm_t, int *) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

Nccl &nccl() {
    static Nccl n;
    if (n.lib) return n;
    n.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!n.lib) n.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!n.lib) return n;
    *(void **)&n.GetUniqueId = dlsym(n.lib, "ncclGetUniqueId");
    *(void **)&n.CommInitRank = dlsym(n.lib, "ncclCommInitRank");
    *(void **)&n.CommDestroy = dlsym(n.lib, "ncclCommDestroy");
    *(void **)&n.CommCount = dlsym(n.lib, "ncclCommCount");
    *(void **)&n.AllReduce = dlsym(n.lib, "ncclAllReduce");
    *(void **)&n.GetErrorString = dlsym(n.lib, "ncclGetErrorString");
    n.ok = n.GetUniqueId && n.CommInitRank && n.CommDestroy && n.CommCount && n.AllReduce && n.GetErrorString;
    return n;
}

std::map<anvil_rt *, ncclComm_t> &comms() {
    static std::map<anvil_rt *, ncclComm_t> m;
    return m;
}

int collective(void *user, void *device_ptr, long count, void *cuda_stream) {
    ncclComm_t comm = (ncclComm_t)user;
    ncclResult_t r = nccl().AllReduce(device_ptr, device_ptr, (size_t)count, ncclFloat, ncclSum, comm, (cudaStream_t)cuda_stream);
    if (r != ncclSuccess) {
        fprintf(stderr, "anvil: ncclAllReduce failed: %s\n", nccl().GetErrorString(r));
        return 1;
    }
    return 0;
}

}  // namespace

extern "C" int anvil_rt_comm_unique_id(void *id_out, size_t bytes) {
    if (!id_out || bytes < sizeof(ncclUniqueId) || !nccl().ok) return 1;
    ncclUniqueId id;
    if (nccl().GetUniqueId(&id) != ncclSuccess) return 1;
    memcpy(id_out, &id, sizeof id);
    return 0;
}

extern "C" int anvil_rt_comm_init(anvil_rt *rt, int rank, int nranks, const void *unique_id, size_t bytes) {
    if (!rt) return 1;
    if (!nccl().ok) return anvil_rt_set_error(rt, "anvil: libnccl.so.2 could not be loaded");
    if (!unique_id || bytes < sizeof(ncclUniqueId) || rank < 0 || rank >= nranks)
        return anvil_rt_set_error(rt, "anvil: bad arguments to anvil_rt_comm_init");
    setenv("NCCL_ALGO", "Ring", 0);                    // a fixed order of additions for a given number of ranks
    setenv("NCCL_PROTO", "Simple", 0);
    setenv("NCCL_MIN_NCHANNELS", "8", 0);
    setenv("NCCL_MAX_NCHANNELS", "8", 0);
    ncclUniqueId id;
    memcpy(&id, unique_id, sizeof id);
    ncclComm_t comm = nullptr;
    ncclResult_t r = nccl().CommInitRank(&comm, nranks, id, rank);
    if (r != ncclSuccess) {
        char msg[256];
        snprintf(msg, sizeof msg, "anvil: ncclCommInitRank failed: %s", nccl().GetErrorString(r));
        return anvil_rt_set_error(rt, msg);
    }
    auto it = comms().find(rt);
    if (it != comms().end()) nccl().CommDestroy(it->second);
    comms()[rt] = comm;
    anvil_rt_set_allreduce(rt, collective, comm);
    return 0;
}

extern "C" int anvil_rt_comm_nranks(anvil_rt *rt) {
    auto it = comms().find(rt);
    if (it == comms().end()) return 0;
    int n = 0;
    return nccl().CommCount(it->second, &n) == ncclSuccess ? n : 0;
}

extern "C" int anvil_rt_comm_destroy(anvil_rt *rt) {
    auto it = comms().find(rt);
    if (it == comms().end()) return 0;
    nccl().CommDestroy(it->second);
    comms().erase(it);
    anvil_rt_set_allreduce(rt, nullptr, nullptr);
    return 0;
}
