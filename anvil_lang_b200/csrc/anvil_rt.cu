// anvil_rt.cu — libanvil_cuda.so: the runtime behind the C ABI declared in include/anvil_cuda.h.
//
// One context = one device, one stream, one cudaMalloc'd arena. Host-side services (printing,
// shuffle, checkpoints) stage through host memory with explicit copies; the formats follow the
// reference runtime (anvil/backend/anvil_host.h) byte for byte.
#include "anvil_cuda.h"
#include "anvil_rng.h"

#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <zlib.h>

#include <map>
#include <string>
#include <thread>
#include <vector>

struct anvil_graph {
    cudaGraphExec_t exec = nullptr;
    long nodes = 0;
    uint32_t streams_taken = 0;     // host stream numbers consumed by the recorded launches
    uint32_t pending_after = 0;     // host-minus-device stream difference when the recording ended
};

struct anvil_rt {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = true;
    char *arena = nullptr;
    size_t arena_bytes = 0;
    uint32_t seed = 0;
    uint32_t host_stream = 0;       // next stream number (authoritative)
    uint32_t pending = 0;           // host_stream - device copy, in stream order
    double t0 = 0;
    std::string error;
    std::string captured;
    bool capture = false;
    const char *const *fault_messages = nullptr;
    int n_fault_messages = 0;
    bool graphs_on = true;
    int capturing_key = -1;
    uint32_t capture_stream0 = 0;
    std::map<int, anvil_graph> graphs;
    long launches = 0;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    anvil_allreduce_fn allreduce = nullptr;
    void *allreduce_user = nullptr;
    int check = 0;                  // --check: 1 = nan, 2 = nan or infinity, scanned after every launch unit
    bool profile = false;           // time every launch unit (graphs off) and report at the end of the program
    std::map<int, std::pair<double, long>> prof;      // slot -> (milliseconds, calls)
    std::vector<int> prof_order;    // slots in the order they first ran
    cudaEvent_t pe0 = nullptr, pe1 = nullptr;
    char *stage[2] = {nullptr, nullptr};        // pinned staging buffers for large copies from / to pageable host memory
    cudaEvent_t stage_ev[2] = {nullptr, nullptr};
    // second stream: kernels whose results nothing in the rest of their launch run needs (parameter updates of small
    // tensors) run beside the kernels that follow them; fork / join are event edges, which a stream capture records
    // as graph dependencies
    cudaStream_t side = nullptr;
    cudaStream_t current = nullptr;             // what launches go to; nullptr = `stream`
    cudaEvent_t fork_ev = nullptr, join_ev = nullptr;
    bool forked = false;
    bool side_on = true;
};

static double now_seconds() {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec + ts.tv_nsec * 1e-9;
}

static int fail(anvil_rt *rt, const char *fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (rt) rt->error = buf;
    return 1;
}

#define CK(rt, call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) \
    return fail((rt), "anvil: CUDA error: %s (%s)", cudaGetErrorString(e_), #call); } while (0)

// ---------------------------------------------------------------------------- small kernels
__global__ void k_set_u32(uint32_t *p, uint32_t v) { *p = v; }
__global__ void k_add_u32(uint32_t *p, uint32_t v) { *p += v; }
__global__ void k_iota(int *p, long n) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) p[i] = (int)i;
}

// ---------------------------------------------------------------------------- context
extern "C" anvil_rt *anvil_rt_create(int device) {
    anvil_rt *rt = new anvil_rt();
    rt->device = device;
    rt->t0 = now_seconds();
    if (cudaSetDevice(device) != cudaSuccess ||
        cudaStreamCreateWithFlags(&rt->stream, cudaStreamNonBlocking) != cudaSuccess) {
        rt->error = std::string("anvil: CUDA error: ") + cudaGetErrorString(cudaGetLastError());
        rt->stream = nullptr;
    }
    if (rt->stream && (cudaStreamCreateWithFlags(&rt->side, cudaStreamNonBlocking) != cudaSuccess ||
                       cudaEventCreateWithFlags(&rt->fork_ev, cudaEventDisableTiming) != cudaSuccess ||
                       cudaEventCreateWithFlags(&rt->join_ev, cudaEventDisableTiming) != cudaSuccess)) {
        cudaGetLastError();
        rt->side = nullptr;                      // no second stream: everything runs on the first
    }
    return rt;
}

extern "C" void anvil_rt_destroy(anvil_rt *rt) {
    if (!rt) return;
    cudaSetDevice(rt->device);
    if (rt->stream) cudaStreamSynchronize(rt->stream);
    anvil_rt_comm_destroy(rt);
    for (auto &g : rt->graphs) if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
    if (rt->arena) cudaFree(rt->arena);
    if (rt->ev0) { cudaEventDestroy(rt->ev0); cudaEventDestroy(rt->ev1); }
    if (rt->pe0) { cudaEventDestroy(rt->pe0); cudaEventDestroy(rt->pe1); }
    for (int i = 0; i < 2; i++) { if (rt->stage[i]) cudaFreeHost(rt->stage[i]); if (rt->stage_ev[i]) cudaEventDestroy(rt->stage_ev[i]); }
    if (rt->side) { cudaStreamSynchronize(rt->side); cudaStreamDestroy(rt->side); }
    if (rt->fork_ev) cudaEventDestroy(rt->fork_ev);
    if (rt->join_ev) cudaEventDestroy(rt->join_ev);
    if (rt->stream && rt->own_stream) cudaStreamDestroy(rt->stream);
    delete rt;
}

extern "C" int anvil_rt_arena(anvil_rt *rt, size_t bytes) {
    if (!rt->stream) return 1;
    CK(rt, cudaSetDevice(rt->device));
    if (rt->arena) { CK(rt, cudaFree(rt->arena)); rt->arena = nullptr; }
    if (bytes < ANVIL_RT_HEADER_BYTES) bytes = ANVIL_RT_HEADER_BYTES;
    cudaError_t e = cudaMalloc((void **)&rt->arena, bytes);
    if (e != cudaSuccess) { rt->arena = nullptr; return fail(rt, "anvil: out of memory (%zu bytes)", bytes); }
    rt->arena_bytes = bytes;
    CK(rt, cudaMemsetAsync(rt->arena, 0, bytes, rt->stream));
    rt->pending = rt->host_stream;          // the device copy of the stream counter restarts at 0
    return 0;
}

extern "C" void *anvil_rt_ptr(anvil_rt *rt, size_t off) { return rt->arena + off; }
extern "C" size_t anvil_rt_arena_bytes(anvil_rt *rt) { return rt->arena_bytes; }
extern "C" void *anvil_rt_stream(anvil_rt *rt) { return (void *)(rt->current ? rt->current : rt->stream); }

// The next launches go to the second stream, ordered after everything issued on the first so far. With --profile or
// --check (every launch unit is timed or scanned on the first stream) or without a second stream this is a no-op.
extern "C" int anvil_rt_fork(anvil_rt *rt) {
    if (!rt->side || !rt->side_on || rt->profile || rt->check) return 0;
    CK(rt, cudaEventRecord(rt->fork_ev, rt->stream));
    CK(rt, cudaStreamWaitEvent(rt->side, rt->fork_ev, 0));
    rt->current = rt->side;
    rt->forked = true;
    return 0;
}
extern "C" int anvil_rt_back(anvil_rt *rt) { rt->current = nullptr; return 0; }
// The first stream waits for what the second one was given since the last join.
extern "C" int anvil_rt_join(anvil_rt *rt) {
    rt->current = nullptr;
    if (!rt->forked) return 0;
    rt->forked = false;
    CK(rt, cudaEventRecord(rt->join_ev, rt->side));
    CK(rt, cudaStreamWaitEvent(rt->stream, rt->join_ev, 0));
    return 0;
}
extern "C" int anvil_rt_side_stream(anvil_rt *rt, int on) { rt->side_on = on != 0; return 0; }
extern "C" int anvil_rt_use_stream(anvil_rt *rt, void *s) {
    if (rt->stream && rt->own_stream) { cudaStreamSynchronize(rt->stream); cudaStreamDestroy(rt->stream); }
    rt->stream = (cudaStream_t)s;
    rt->own_stream = false;
    return 0;
}
extern "C" const char *anvil_rt_last_error(anvil_rt *rt) { return rt->error.c_str(); }
extern "C" int anvil_rt_set_error(anvil_rt *rt, const char *m) { rt->error = m ? m : ""; return 1; }

static int in_range(anvil_rt *rt, size_t off, size_t bytes) {
    if (!rt->arena || off > rt->arena_bytes || bytes > rt->arena_bytes - off)
        return fail(rt, "anvil: arena access out of range (offset %zu, %zu bytes, arena %zu)", off, bytes, rt->arena_bytes);
    return 0;
}

// ---------------------------------------------------------------------------- data movement
extern "C" int anvil_rt_h2d(anvil_rt *rt, size_t off, const void *src, size_t bytes) {
    if (in_range(rt, off, bytes)) return 1;
    CK(rt, cudaMemcpyAsync(rt->arena + off, src, bytes, cudaMemcpyHostToDevice, rt->stream));
    CK(rt, cudaStreamSynchronize(rt->stream));
    return 0;
}
extern "C" int anvil_rt_d2h(anvil_rt *rt, void *dst, size_t off, size_t bytes) {
    if (in_range(rt, off, bytes)) return 1;
    CK(rt, cudaMemcpyAsync(dst, rt->arena + off, bytes, cudaMemcpyDeviceToHost, rt->stream));
    CK(rt, cudaStreamSynchronize(rt->stream));
    return 0;
}
extern "C" int anvil_rt_h2d_async(anvil_rt *rt, size_t off, const void *src, size_t bytes) {
    if (in_range(rt, off, bytes)) return 1;
    CK(rt, cudaMemcpyAsync(rt->arena + off, src, bytes, cudaMemcpyHostToDevice, rt->stream));
    return 0;
}
// Device-to-device copy into the arena from memory another library owns (a `__cuda_array_interface__`
// argument of anvil.function): waits for the producer first — its stream when the interface names one
// (`producer_stream` != 0), the whole device otherwise — then copies on the program's stream.
extern "C" int anvil_rt_d2d_async(anvil_rt *rt, size_t off, const void *src_device, size_t bytes, void *producer_stream) {
    if (in_range(rt, off, bytes)) return 1;
    if (producer_stream) CK(rt, cudaStreamSynchronize((cudaStream_t)producer_stream));
    else CK(rt, cudaDeviceSynchronize());
    CK(rt, cudaMemcpyAsync(rt->arena + off, src_device, bytes, cudaMemcpyDeviceToDevice, rt->stream));
    return 0;
}

extern "C" int anvil_rt_d2h_async(anvil_rt *rt, void *dst, size_t off, size_t bytes) {
    if (in_range(rt, off, bytes)) return 1;
    CK(rt, cudaMemcpyAsync(dst, rt->arena + off, bytes, cudaMemcpyDeviceToHost, rt->stream));
    return 0;
}
// Large copies between the arena and PAGEABLE host memory (the arrays an `anvil.function` caller hands over): a plain
// cudaMemcpyAsync stages them through the driver's own bounce buffer at about 5 GB/s. Here the copy is cut into 8 MiB
// chunks that go through two pinned buffers: host threads fill (or drain) one while the DMA engine moves the other.
static const size_t STAGE_BYTES = 8u << 20;
static const int STAGE_THREADS = 4;
static void parallel_copy(char *dst, const char *src, size_t n) {
    if (n < (1u << 20)) { memcpy(dst, src, n); return; }
    std::thread th[STAGE_THREADS];
    const size_t part = (n / STAGE_THREADS + 63) / 64 * 64;
    for (int i = 0; i < STAGE_THREADS; i++) {
        const size_t lo = (size_t)i * part, hi = lo + part < n ? lo + part : n;
        th[i] = std::thread([=] { if (lo < hi) memcpy(dst + lo, src + lo, hi - lo); });
    }
    for (auto &t : th) t.join();
}
static int ensure_stage(anvil_rt *rt) {
    for (int i = 0; i < 2; i++) {
        if (!rt->stage[i]) CK(rt, cudaMallocHost((void **)&rt->stage[i], STAGE_BYTES));
        if (!rt->stage_ev[i]) CK(rt, cudaEventCreateWithFlags(&rt->stage_ev[i], cudaEventDisableTiming));
    }
    return 0;
}
extern "C" int anvil_rt_h2d_staged(anvil_rt *rt, size_t off, const void *src, size_t bytes) {
    if (in_range(rt, off, bytes)) return 1;
    if (bytes < 2 * STAGE_BYTES) return anvil_rt_h2d_async(rt, off, src, bytes);
    if (ensure_stage(rt)) return 1;
    int i = 0;
    for (size_t done = 0; done < bytes; done += STAGE_BYTES, i ^= 1) {
        const size_t n = bytes - done < STAGE_BYTES ? bytes - done : STAGE_BYTES;
        CK(rt, cudaEventSynchronize(rt->stage_ev[i]));                  // the copy that last used this buffer has finished
        parallel_copy(rt->stage[i], (const char *)src + done, n);
        CK(rt, cudaMemcpyAsync(rt->arena + off + done, rt->stage[i], n, cudaMemcpyHostToDevice, rt->stream));
        CK(rt, cudaEventRecord(rt->stage_ev[i], rt->stream));
    }
    return 0;
}
// The result is in `dst` when the call returns (unlike anvil_rt_d2h_async).
extern "C" int anvil_rt_d2h_staged(anvil_rt *rt, void *dst, size_t off, size_t bytes) {
    if (in_range(rt, off, bytes)) return 1;
    if (bytes < 2 * STAGE_BYTES) { if (anvil_rt_d2h_async(rt, dst, off, bytes)) return 1; return anvil_rt_sync(rt); }
    if (ensure_stage(rt)) return 1;
    const size_t chunks = (bytes + STAGE_BYTES - 1) / STAGE_BYTES;
    for (size_t c = 0; c <= chunks; c++) {                              // chunk c is copied out while chunk c - 1 is drained
        if (c < chunks) {
            const size_t n = bytes - c * STAGE_BYTES < STAGE_BYTES ? bytes - c * STAGE_BYTES : STAGE_BYTES;
            CK(rt, cudaMemcpyAsync(rt->stage[c & 1], rt->arena + off + c * STAGE_BYTES, n, cudaMemcpyDeviceToHost, rt->stream));
            CK(rt, cudaEventRecord(rt->stage_ev[c & 1], rt->stream));
        }
        if (c > 0) {
            const size_t p = c - 1, n = bytes - p * STAGE_BYTES < STAGE_BYTES ? bytes - p * STAGE_BYTES : STAGE_BYTES;
            CK(rt, cudaEventSynchronize(rt->stage_ev[p & 1]));
            parallel_copy((char *)dst + p * STAGE_BYTES, rt->stage[p & 1], n);
        }
    }
    return 0;
}
extern "C" int anvil_rt_zero(anvil_rt *rt, size_t off, size_t bytes) {
    if (in_range(rt, off, bytes)) return 1;
    CK(rt, cudaMemsetAsync(rt->arena + off, 0, bytes, rt->stream));
    if (off <= ANVIL_RT_STREAM_OFF && off + bytes >= ANVIL_RT_STREAM_OFF + 4)
        rt->pending = rt->host_stream;      // the device copy of the stream counter is 0 again
    return 0;
}
extern "C" int anvil_rt_sync(anvil_rt *rt) {
    CK(rt, cudaStreamSynchronize(rt->stream));
    return 0;
}
extern "C" void *anvil_rt_host_alloc(size_t bytes) {
    void *p = nullptr;
    if (cudaMallocHost(&p, bytes ? bytes : 1) != cudaSuccess) return nullptr;
    return p;
}
extern "C" void anvil_rt_host_free(void *p) { if (p) cudaFreeHost(p); }

// ---------------------------------------------------------------------------- scalars
extern "C" int anvil_rt_set_i32(anvil_rt *rt, size_t off, int32_t v) {
    if (in_range(rt, off, 4)) return 1;
    k_set_u32<<<1, 1, 0, rt->stream>>>((uint32_t *)(rt->arena + off), (uint32_t)v);
    rt->launches++;
    CK(rt, cudaGetLastError());
    return 0;
}
extern "C" int anvil_rt_set_f32(anvil_rt *rt, size_t off, float v) {
    uint32_t u; memcpy(&u, &v, 4);
    return anvil_rt_set_i32(rt, off, (int32_t)u);
}
extern "C" int anvil_rt_add_i32(anvil_rt *rt, size_t off, int32_t d) {
    if (in_range(rt, off, 4)) return 1;
    k_add_u32<<<1, 1, 0, rt->stream>>>((uint32_t *)(rt->arena + off), (uint32_t)d);
    rt->launches++;
    CK(rt, cudaGetLastError());
    return 0;
}
extern "C" int anvil_rt_read_i32(anvil_rt *rt, size_t off, int32_t *out) { return anvil_rt_d2h(rt, out, off, 4); }
extern "C" int anvil_rt_read_f32(anvil_rt *rt, size_t off, float *out) { return anvil_rt_d2h(rt, out, off, 4); }

// ---------------------------------------------------------------------------- random numbers
extern "C" void anvil_rt_seed(anvil_rt *rt, uint32_t seed) {
    rt->seed = seed;
    anvil_rt_set_stream(rt, 0);
}
extern "C" uint32_t anvil_rt_get_seed(anvil_rt *rt) { return rt->seed; }
extern "C" uint32_t anvil_rt_get_stream(anvil_rt *rt) { return rt->host_stream; }
extern "C" void anvil_rt_set_stream(anvil_rt *rt, uint32_t s) {
    rt->pending += s - rt->host_stream;     // modulo 2^32, like the counters themselves
    rt->host_stream = s;
}
extern "C" uint32_t anvil_rt_next_stream_delta(anvil_rt *rt) {
    uint32_t d = rt->pending;
    rt->host_stream++;
    rt->pending++;
    return d;
}
extern "C" int anvil_rt_stream_commit(anvil_rt *rt) {
    if (rt->pending == 0 || !rt->arena) return 0;
    k_add_u32<<<1, 1, 0, rt->stream>>>((uint32_t *)(rt->arena + ANVIL_RT_STREAM_OFF), rt->pending);
    rt->launches++;
    CK(rt, cudaGetLastError());
    rt->pending = 0;
    return 0;
}
extern "C" uint32_t anvil_rt_rand_bits(uint32_t idx, uint32_t stream, uint32_t salt, uint32_t seed) {
    return anvil_rand_bits(idx, stream, salt, seed);
}
extern "C" float anvil_rt_rand(uint32_t idx, uint32_t stream, uint32_t salt, uint32_t seed, int open_low) {
    return anvil_rand(idx, stream, salt, seed, open_low);
}

// ---------------------------------------------------------------------------- runtime calls
extern "C" int anvil_rt_iota(anvil_rt *rt, size_t off, long n) {
    if (in_range(rt, off, 4 * (size_t)n)) return 1;
    if (n <= 0) return 0;
    long blocks = (n + 255) / 256;
    k_iota<<<(unsigned)(blocks > 1184 ? 1184 : blocks), 256, 0, rt->stream>>>((int *)(rt->arena + off), n);
    rt->launches++;
    CK(rt, cudaGetLastError());
    return 0;
}

// Fisher-Yates with the draws of anvil/backend/anvil_host.h:269-276. The swaps depend on one
// another, so the permutation is staged through host memory (240 KB for 60000 entries).
extern "C" int anvil_rt_shuffle(anvil_rt *rt, size_t off, long n) {
    uint32_t stream = rt->host_stream;
    anvil_rt_set_stream(rt, stream + 1);
    if (n < 2) return 0;
    std::vector<int> p((size_t)n);
    if (anvil_rt_d2h(rt, p.data(), off, 4 * (size_t)n)) return 1;
    for (long k = 0; k < n - 1; k++) {
        long i = n - 1 - k;
        long j = anvil_rand_bits((uint32_t)k, stream, 7, rt->seed) % (uint32_t)(i + 1);
        int t = p[i]; p[i] = p[j]; p[j] = t;
    }
    return anvil_rt_h2d(rt, off, p.data(), 4 * (size_t)n);
}

extern "C" int anvil_rt_nonzero(anvil_rt *rt, size_t src_off, long n, size_t dst_off, long size) {
    std::vector<int> flags((size_t)(n > 0 ? n : 1)), out((size_t)(size > 0 ? size : 1));
    if (anvil_rt_d2h(rt, flags.data(), src_off, 4 * (size_t)n)) return 1;
    long k = 0;
    for (long i = 0; i < n && k < size; i++) if (flags[i]) out[k++] = (int)i;
    for (; k < size; k++) out[k] = -1;
    return anvil_rt_h2d(rt, dst_off, out.data(), 4 * (size_t)size);
}

extern "C" int anvil_rt_clock(anvil_rt *rt, size_t off) {
    if (anvil_rt_sync(rt)) return 1;
    return anvil_rt_set_f32(rt, off, (float)(now_seconds() - rt->t0));
}

// Checkpoints: "EINW", u32 version 2, u64 count, count u64 keys, then raw little-endian payloads
// (anvil/backend/anvil_host.h:237-266; anvil/interp.py:341-372). Version 1 stored counts only.
extern "C" int anvil_rt_save(anvil_rt *rt, const char *path, const anvil_rt_ckpt *tab, long n) {
    FILE *f = fopen(path, "wb");
    if (!f) { fprintf(stderr, "anvil: cannot write %s\n", path); return 0; }
    uint64_t head = 0x00000002574E4945ull, cnt = (uint64_t)n;
    fwrite(&head, 8, 1, f); fwrite(&cnt, 8, 1, f);
    for (long i = 0; i < n; i++) fwrite(&tab[i].key, 8, 1, f);
    int rc = 0;
    for (long i = 0; i < n && !rc; i++) {
        size_t count = (size_t)(tab[i].key & 0xFFFFFFFFull);
        std::vector<char> host(4 * count + 4);
        rc = anvil_rt_d2h(rt, host.data(), tab[i].off, 4 * count);
        if (!rc) fwrite(host.data(), 4, count, f);
    }
    fclose(f);
    return rc;
}

extern "C" int anvil_rt_load(anvil_rt *rt, const char *path, const anvil_rt_ckpt *tab, long n, float *okp) {
    *okp = 0.0f;
    FILE *f = fopen(path, "rb");
    if (!f) return 0;
    uint64_t head = 0, cnt = 0, total = 0;
    int ok = fread(&head, 8, 1, f) == 1 && (head == 0x00000002574E4945ull || head == 0x00000001574E4945ull)
             && fread(&cnt, 8, 1, f) == 1 && cnt == (uint64_t)n;
    uint64_t mask = head == 0x00000002574E4945ull ? ~0ull : 0xFFFFFFFFull;
    for (long i = 0; ok && i < n; i++) {
        uint64_t c;
        ok = fread(&c, 8, 1, f) == 1 && c == (tab[i].key & mask);
        total += tab[i].key & 0xFFFFFFFFull;
    }
    if (ok) { fseek(f, 0, SEEK_END); ok = ftell(f) == (long)(16 + 8 * n + 4 * total); fseek(f, 16 + 8 * n, SEEK_SET); }
    int rc = 0;
    for (long i = 0; ok && i < n && !rc; i++) {
        size_t count = (size_t)(tab[i].key & 0xFFFFFFFFull);
        std::vector<char> host(4 * count + 4);
        ok = fread(host.data(), 4, count, f) == count;
        if (ok) rc = anvil_rt_h2d(rt, tab[i].off, host.data(), 4 * count);
    }
    fclose(f);
    if (!rc && ok) *okp = 1.0f;
    return rc;
}

extern "C" int anvil_rt_save_npy(anvil_rt *rt, const char *path, const unsigned char *header, long hlen,
                                 size_t off, long bytes) {
    std::vector<char> host((size_t)bytes + 4);
    if (anvil_rt_d2h(rt, host.data(), off, (size_t)bytes)) return 1;
    FILE *f = fopen(path, "wb");
    if (!f) { fprintf(stderr, "anvil: cannot write %s\n", path); return 0; }
    fwrite(header, 1, (size_t)hlen, f);
    fwrite(host.data(), 1, (size_t)bytes, f);
    fclose(f);
    return 0;
}

static void emit(anvil_rt *rt, const char *s, int to_stderr);

// ANVIL_DATA, when set, replaces the directory of every data file (anvil_host.h:134-141).
static std::string data_path(const char *path) {
    const char *dir = getenv("ANVIL_DATA");
    if (!dir || !*dir) return path;
    const char *name = strrchr(path, '/');
    return std::string(dir) + "/" + (name ? name + 1 : path);
}
static const char *const BAD_SHAPE = "anvil: data file %s does not have the shape this program was compiled for";

// An IDX file (plain or gzip): `header` bytes are skipped, then n unsigned bytes become f32 or i32
// values (anvil_host.h:143-156; anvil/interp.py:243-251).
extern "C" int anvil_rt_load_idx(anvil_rt *rt, const char *path0, size_t off, long n, long header, int is_int) {
    const std::string path = data_path(path0);
    gzFile f = gzopen(path.c_str(), "rb");
    if (!f) return fail(rt, "anvil: cannot open data file %s", path.c_str());
    std::vector<unsigned char> raw((size_t)(n > 0 ? n : 1)), skip((size_t)(header > 0 ? header : 1));
    const bool ok = gzread(f, skip.data(), (unsigned)header) == (int)header && gzread(f, raw.data(), (unsigned)n) == (int)n;
    gzclose(f);
    if (!ok) return fail(rt, BAD_SHAPE, path.c_str());
    std::vector<uint32_t> out((size_t)(n > 0 ? n : 1));
    for (long i = 0; i < n; i++) {
        if (is_int) { int32_t v = raw[i]; memcpy(&out[i], &v, 4); }
        else { float v = (float)raw[i]; memcpy(&out[i], &v, 4); }
    }
    return anvil_rt_h2d(rt, off, out.data(), 4 * (size_t)n);
}

static bool read_file(const std::string &path, std::string &text) {
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) return false;
    char chunk[1 << 16];
    size_t got;
    while ((got = fread(chunk, 1, sizeof chunk, f)) > 0) text.append(chunk, got);
    fclose(f);
    return true;
}

// "[+-] digit ..." or "[+-] . digit ..." (anvil_host.h:172-177)
static bool number_starts(const char *p) {
    if (*p == '+' || *p == '-') p++;
    if (*p == '.') p++;
    return *p >= '0' && *p <= '9';
}

// The first n numbers of a text file after `skip` lines, whatever separates them (anvil_host.h:179-190).
extern "C" int anvil_rt_load_csv(anvil_rt *rt, const char *path0, size_t off, long n, long skip) {
    const std::string path = data_path(path0);
    std::string text;
    if (!read_file(path, text)) return fail(rt, "anvil: cannot open data file %s", path.c_str());
    const char *p = text.c_str();
    for (long s = 0; s < skip && *p; p++) if (*p == '\n') s++;
    std::vector<float> out((size_t)(n > 0 ? n : 1));
    long got = 0;
    while (got < n && *p) {
        if (number_starts(p)) { char *end; out[got++] = strtof(p, &end); p = end; }
        else p++;
    }
    if (got < n) return fail(rt, BAD_SHAPE, path.c_str());
    return anvil_rt_h2d(rt, off, out.data(), 4 * (size_t)n);
}

// Exactly n bytes, each becoming one i32 (anvil_host.h:192-197).
extern "C" int anvil_rt_load_bytes(anvil_rt *rt, const char *path0, size_t off, long n) {
    const std::string path = data_path(path0);
    std::string text;
    if (!read_file(path, text)) return fail(rt, "anvil: cannot open data file %s", path.c_str());
    if ((long)text.size() != n) return fail(rt, BAD_SHAPE, path.c_str());
    std::vector<int32_t> out((size_t)(n > 0 ? n : 1));
    for (long i = 0; i < n; i++) out[i] = (unsigned char)text[i];
    return anvil_rt_h2d(rt, off, out.data(), 4 * (size_t)n);
}

// One line of standard input: its first decimal number (NaN if it has none) goes to the f32 at `off`;
// *eof = 1 at the end of the input, after a newline has been printed (anvil_host.h:286-300).
extern "C" int anvil_rt_input(anvil_rt *rt, size_t off, int *eof) {
    char line[256];
    anvil_rt_flush(rt);
    *eof = 0;
    if (!fgets(line, sizeof line, stdin)) { emit(rt, "\n", 0); *eof = 1; return 0; }
    float v = NAN;
    for (char *p = line; *p; p++) {
        if (number_starts(p)) {
            char *q = p;
            if (*q == '+' || *q == '-') q++;
            if (q[0] == '0' && (q[1] == 'x' || q[1] == 'X')) q[1] = 0;          // decimal only
            v = strtof(p, nullptr);
            break;
        }
    }
    return anvil_rt_set_f32(rt, off, v);
}

// n values from byte `offset` of a NumPy (or safetensors, kind + 16) file converted to 32 bits;
// kinds: 0 f32, 1 f64, 2 f16, 3 i32, 4 i64, 5 u8, 6 i8, 7 u16, 8 i16 (anvil_host.h:189-220).
extern "C" int anvil_rt_load_npy(anvil_rt *rt, const char *path0, size_t off, long n, long offset, int kind, int size) {
    const std::string path_s = data_path(path0);          // ANVIL_DATA relocates these files too (anvil_host.h:199)
    const char *path = path_s.c_str();
    FILE *f = fopen(path, "rb");
    if (!f) return fail(rt, "anvil: cannot open data file %s", path);
    fseek(f, offset, SEEK_SET);
    long extra = (kind & 16) ? 0 : 1;
    kind &= 15;
    std::vector<unsigned char> raw((size_t)n * size + 1);
    long got = (long)fread(raw.data(), 1, (size_t)n * size + extra, f);
    fclose(f);
    if (got != n * size)
        return fail(rt, "anvil: data file %s does not have the shape this program was compiled for", path);
    std::vector<uint32_t> out((size_t)(n > 0 ? n : 1));
    for (long i = 0; i < n; i++) {
        const unsigned char *p = raw.data() + (size_t)i * size;
        float fv = 0; int32_t iv = 0; bool isf = kind <= 2;
        double dv; int64_t lv; int16_t sv; uint16_t uv;
        switch (kind) {
        case 0: memcpy(&fv, p, 4); break;
        case 1: memcpy(&dv, p, 8); fv = (float)dv; break;
        case 2: { memcpy(&uv, p, 2); int e = (uv >> 10) & 31, m = uv & 1023;
                  float v = e == 0 ? ldexpf((float)m, -24) : e == 31 ? (m ? NAN : INFINITY) : ldexpf((float)(m | 1024), e - 25);
                  fv = (uv & 0x8000) ? -v : v; break; }
        case 3: memcpy(&iv, p, 4); break;
        case 4: memcpy(&lv, p, 8); iv = (int32_t)lv; break;
        case 5: iv = p[0]; break;
        case 6: iv = (signed char)p[0]; break;
        case 7: memcpy(&uv, p, 2); iv = uv; break;
        default: memcpy(&sv, p, 2); iv = sv; break;
        }
        if (isf) memcpy(&out[i], &fv, 4); else memcpy(&out[i], &iv, 4);
    }
    return anvil_rt_h2d(rt, off, out.data(), 4 * (size_t)n);
}

// ---------------------------------------------------------------------------- output
static void emit(anvil_rt *rt, const char *s, int to_stderr) {
    if (rt->capture && !to_stderr) rt->captured += s;
    else if (to_stderr) { fflush(stdout); fputs(s, stderr); }
    else fputs(s, stdout);
}

static void emitf(anvil_rt *rt, int to_stderr, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    emit(rt, buf, to_stderr);
}

// %-formatting of a double the way Python's `fmt % v` prints it: identical to C except that C may
// print the sign of a nan.
static void emit_double(anvil_rt *rt, int to_stderr, const char *fmt, double v) {
    if (v != v) {
        char buf[512];
        snprintf(buf, sizeof buf, fmt, (double)NAN);
        std::string s(buf);
        size_t at = s.find("-nan");
        if (at != std::string::npos) s.replace(at, 4, "nan");
        emit(rt, s.c_str(), to_stderr);
        return;
    }
    emitf(rt, to_stderr, fmt, v);
}

static void emit_f32(anvil_rt *rt, int to_stderr, float v) {     // anvil_host.h:76-80
    double a = fabs((double)v);
    if (v == 0 || v != v || (a >= 1e-4 && a < 1e6)) emit_double(rt, to_stderr, "%.4f", (double)v);
    else emit_double(rt, to_stderr, "%.4e", (double)v);
}

extern "C" int anvil_rt_capture(anvil_rt *rt, int on) { rt->capture = on != 0; if (on) rt->captured.clear(); return 0; }
extern "C" const char *anvil_rt_captured(anvil_rt *rt) { return rt->captured.c_str(); }
extern "C" int anvil_rt_flush(anvil_rt *rt) { (void)rt; fflush(stdout); return 0; }
extern "C" int anvil_rt_print_text(anvil_rt *rt, const char *text, int to_stderr) { emit(rt, text, to_stderr); return 0; }

extern "C" int anvil_rt_print_scalar(anvil_rt *rt, size_t off, int is_int, const char *fmt, int fmt_is_int, int to_stderr) {
    uint32_t raw;
    if (anvil_rt_d2h(rt, &raw, off, 4)) return 1;
    int32_t iv; float fv;
    memcpy(&iv, &raw, 4); memcpy(&fv, &raw, 4);
    if (fmt && *fmt) {
        // Python's `fmt % value`: an i32 buffer (or a %d conversion) prints int(value)
        // (anvil/interp.py:218-225); a float conversion of an int value still takes a double here.
        double as_double = (is_int || fmt_is_int) ? (double)(is_int ? iv : (int)fv) : (double)fv;
        if (fmt_is_int) emitf(rt, to_stderr, fmt, is_int ? iv : (int)fv);
        else emit_double(rt, to_stderr, fmt, as_double);
    } else if (is_int) emitf(rt, to_stderr, "%d", iv);
    else emit_f32(rt, to_stderr, fv);
    return 0;
}

static void print_rec(anvil_rt *rt, const void *data, int is_int, int rank, const long *dims, const long *strides,
                      long off, int d, int summarize) {
    long n = dims[d];
    emit(rt, "[", 0);
    long idx[7]; int cnt = 0;
    if (summarize && n > 6) { idx[0] = 0; idx[1] = 1; idx[2] = 2; idx[3] = -1; idx[4] = n - 3; idx[5] = n - 2; idx[6] = n - 1; cnt = 7; }
    for (long k = 0; k < (cnt ? cnt : n); k++) {
        long i = cnt ? idx[k] : k;
        if (k) {
            if (d == rank - 1) emit(rt, ", ", 0);
            else { emit(rt, ",\n", 0); for (int s = 0; s <= d; s++) emit(rt, " ", 0); }
        }
        if (i < 0) { emit(rt, "...", 0); continue; }
        if (d == rank - 1) {
            if (is_int) emitf(rt, 0, "%d", ((const int *)data)[off + i]);
            else emit_f32(rt, 0, ((const float *)data)[off + i]);
        } else {
            print_rec(rt, data, is_int, rank, dims, strides, off + i * strides[d], d + 1, summarize);
        }
    }
    emit(rt, "]", 0);
}

// Nested brackets; more than 1000 elements are summarised as the first and last three of every
// dimension longer than 6 (anvil_host.h:82-111; anvil/interp.py:89-115).
extern "C" int anvil_rt_print_tensor(anvil_rt *rt, size_t off, int is_int, int rank, const long *dims) {
    long strides[16], numel = 1;
    for (int d = rank - 1; d >= 0; d--) { strides[d] = numel; numel *= dims[d]; }
    std::vector<uint32_t> host((size_t)(numel > 0 ? numel : 1));
    if (anvil_rt_d2h(rt, host.data(), off, 4 * (size_t)(numel > 0 ? numel : 1))) return 1;
    if (rank == 0) {
        if (is_int) emitf(rt, 0, "%d", *(const int *)host.data());
        else emit_f32(rt, 0, *(const float *)host.data());
        return 0;
    }
    if (numel == 0) { emit(rt, "[]", 0); return 0; }
    print_rec(rt, host.data(), is_int, rank, dims, strides, 0, 0, numel > 1000);
    return 0;
}

extern "C" int anvil_rt_print_pick(anvil_rt *rt, size_t off, const char *const *choices, int n, int to_stderr) {
    int32_t k;
    if (anvil_rt_d2h(rt, &k, off, 4)) return 1;
    emit(rt, k >= 0 && k < n ? choices[k] : "?", to_stderr);
    return 0;
}

extern "C" int anvil_rt_print_chars(anvil_rt *rt, size_t off, long n) {
    std::vector<int> codes((size_t)(n > 0 ? n : 1));
    if (anvil_rt_d2h(rt, codes.data(), off, 4 * (size_t)n)) return 1;
    std::string s;
    for (long i = 0; i < n; i++) s.push_back((char)(codes[i] & 0xff));
    emit(rt, s.c_str(), 0);
    return 0;
}

extern "C" int anvil_rt_show(anvil_rt *rt, size_t off, long rows, long cols, const char *const *glyphs, int n) {
    std::vector<int> grid((size_t)(rows * cols > 0 ? rows * cols : 1));
    if (anvil_rt_d2h(rt, grid.data(), off, 4 * (size_t)(rows * cols))) return 1;
    for (long r = 0; r < rows; r++) {
        for (long c = 0; c < cols; c++) {
            int v = grid[r * cols + c];
            emit(rt, v >= 0 && v < n ? glyphs[v] : "?", 0);
        }
        emit(rt, "\n", 0);
    }
    return 0;
}

// ---------------------------------------------------------------------------- faults
extern "C" int anvil_rt_fault_messages(anvil_rt *rt, const char *const *messages, int n) {
    rt->fault_messages = messages;
    rt->n_fault_messages = n;
    return 0;
}

extern "C" int anvil_rt_check_faults(anvil_rt *rt) {
    struct { int code; int pad; long long value; } f;
    if (anvil_rt_d2h(rt, &f, ANVIL_RT_FAULT_OFF, sizeof f)) return 1;
    uint32_t status = 0;
    if (anvil_rt_d2h(rt, &status, ANVIL_RT_STATUS_OFF, 4)) return 1;
    if (status) {
        fflush(stdout);
        return fail(rt, "anvil: runtime error: a kernel gave up waiting on a barrier (status 0x%x)", status);
    }
    if (!f.code) return 0;
    const char *m = (f.code > 0 && f.code < rt->n_fault_messages && rt->fault_messages[f.code])
                        ? rt->fault_messages[f.code] : "index out of bounds";
    fflush(stdout);
    return fail(rt, "anvil: runtime error: %s (got %lld)", m, f.value);
}

extern "C" int anvil_rt_oob(anvil_rt *rt, const char *message, long long value) {
    fflush(stdout);
    return fail(rt, "anvil: runtime error: %s (got %lld)", message, value);
}

// ---------------------------------------------------------------------------- launch-sequence capture
extern "C" void anvil_rt_graphs(anvil_rt *rt, int on) { rt->graphs_on = on != 0; }

// ---------------------------------------------------------------------------- --check
// The reference stops at the first nan (or infinity) a kernel writes and says where and by what
// (anvil/interp.py:408-423; anvil/backend/aarch64.py:82-89, 459-481). Here every launch unit of a generated
// program calls check_tensor for each f32 tensor it wrote; a scan kernel keeps the smallest bad index.
__global__ void anvil_scan_bad(const float *__restrict__ p, long n, int mode, unsigned long long *first) {
    unsigned long long best = ~0ull;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const float v = p[i];
        const bool bad = mode == 1 ? (v != v) : !(fabsf(v) <= 3.402823466e38f);
        if (bad) { best = (unsigned long long)i; break; }           // this thread's indices only grow
    }
    if (best != ~0ull) atomicMin(first, best);
}
extern "C" void anvil_rt_check(anvil_rt *rt, int mode) {
    rt->check = mode;
    if (mode) rt->graphs_on = false;
}
extern "C" int anvil_rt_checking(anvil_rt *rt) { return rt->check; }
extern "C" int anvil_rt_check_tensor(anvil_rt *rt, size_t off, long n, const char *name, const long *shape, int rank,
                                     const char *made_by) {
    if (!rt->check || n <= 0) return 0;
    unsigned long long *first = (unsigned long long *)(rt->arena + ANVIL_RT_CHECK_OFF);
    CK(rt, cudaMemsetAsync(first, 0xFF, 8, rt->stream));
    const int blocks = (int)(n / 256 + 1 < 1184 ? n / 256 + 1 : 1184);
    anvil_scan_bad<<<blocks, 256, 0, rt->stream>>>((const float *)(rt->arena + off), n, rt->check, first);
    unsigned long long idx = ~0ull;
    CK(rt, cudaMemcpyAsync(&idx, first, 8, cudaMemcpyDeviceToHost, rt->stream));
    CK(rt, cudaStreamSynchronize(rt->stream));
    if (idx == ~0ull) return 0;
    float v = 0;
    CK(rt, cudaMemcpy(&v, rt->arena + off + 4 * idx, 4, cudaMemcpyDeviceToHost));
    std::string where;
    if (rank > 0) {
        std::vector<long> ix((size_t)rank);
        unsigned long long r = idx;
        for (int d = rank - 1; d >= 0; d--) { ix[d] = (long)(r % (unsigned long long)shape[d]); r /= (unsigned long long)shape[d]; }
        where = " at [";
        for (int d = 0; d < rank; d++) where += (d ? ", " : "") + std::to_string(ix[d]);
        where += "]";
    }
    const char *what = v != v ? "nan" : (v > 0 ? "inf" : "-inf");
    return fail(rt, "anvil: runtime error: --check: %s in `%s`%s\n%s", what, name, where.c_str(), made_by);
}

// ---------------------------------------------------------------------------- --profile
// The reference's native back end times every kernel and prints "time% ms calls kernel" when the program ends
// (anvil/backend/aarch64.py:383-400, 921-927; runtime.s:1590-1671). Here a launch unit (a kernel, its split
// finish, or a fused row group) is bracketed by two CUDA events on the program's stream.
extern "C" void anvil_rt_profile(anvil_rt *rt, int on) {
    rt->profile = on != 0;
    if (on) rt->graphs_on = false;                   // a replayed graph has no per-kernel boundaries
}
extern "C" int anvil_rt_prof_begin(anvil_rt *rt, int slot) {
    if (!rt->profile) return 0;
    (void)slot;
    if (!rt->pe0) { CK(rt, cudaEventCreate(&rt->pe0)); CK(rt, cudaEventCreate(&rt->pe1)); }
    CK(rt, cudaEventRecord(rt->pe0, rt->stream));
    return 0;
}
extern "C" int anvil_rt_prof_end(anvil_rt *rt, int slot) {
    if (!rt->profile) return 0;
    CK(rt, cudaEventRecord(rt->pe1, rt->stream));
    CK(rt, cudaEventSynchronize(rt->pe1));
    float ms = 0;
    CK(rt, cudaEventElapsedTime(&ms, rt->pe0, rt->pe1));
    auto it = rt->prof.find(slot);
    if (it == rt->prof.end()) { rt->prof_order.push_back(slot); it = rt->prof.emplace(slot, std::make_pair(0.0, 0L)).first; }
    it->second.first += ms;
    it->second.second += 1;
    return 0;
}
extern "C" int anvil_rt_profile_report(anvil_rt *rt, const char *const *names, int n) {
    if (!rt->profile || rt->prof_order.empty()) return 0;
    double total = 0;
    for (auto &kv : rt->prof) total += kv.second.first;
    char line[512];
    emit(rt, "\n  time%        ms      calls   kernel\n", 0);
    for (int slot : rt->prof_order) {
        const auto &r = rt->prof[slot];
        snprintf(line, sizeof line, "%6.1f%%  %8.1f  %9lld   %s\n", 100.0 * r.first / (total > 0 ? total : 1.0), r.first,
                 (long long)r.second, slot < n ? names[slot] : "?");
        emit(rt, line, 0);
    }
    snprintf(line, sizeof line, "          %8.1f ms in kernels\n", total);
    emit(rt, line, 0);
    return 0;
}
extern "C" int anvil_rt_profile_get(anvil_rt *rt, int slot, double *milliseconds, long *calls) {
    auto it = rt->prof.find(slot);
    if (it == rt->prof.end()) { *milliseconds = 0; *calls = 0; return 1; }
    *milliseconds = it->second.first;
    *calls = it->second.second;
    return 0;
}
extern "C" long anvil_rt_launch_count(anvil_rt *rt) { return rt->launches; }
extern "C" void anvil_rt_count_launches(anvil_rt *rt, long n) { rt->launches += n; }

extern "C" int anvil_rt_graph_begin(anvil_rt *rt, int key) {
    if (!rt->graphs_on || rt->capturing_key >= 0) return 2;
    // Recorded launches carry their stream deltas by value, so every recording and every replay
    // starts from "device copy == host counter".
    if (anvil_rt_stream_commit(rt)) return -1;
    auto it = rt->graphs.find(key);
    if (it != rt->graphs.end()) {
        if (cudaGraphLaunch(it->second.exec, rt->stream) != cudaSuccess) {
            fail(rt, "anvil: CUDA error: %s (graph launch)", cudaGetErrorString(cudaGetLastError()));
            return -1;
        }
        rt->launches += it->second.nodes;
        rt->host_stream += it->second.streams_taken;
        rt->pending = it->second.pending_after;
        return 0;
    }
    if (cudaStreamBeginCapture(rt->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
        cudaGetLastError();
        return 2;
    }
    rt->capturing_key = key;
    rt->capture_stream0 = rt->host_stream;
    return 1;
}

extern "C" int anvil_rt_graph_end(anvil_rt *rt, int key) {
    if (rt->capturing_key != key) return fail(rt, "anvil: graph_end without a matching graph_begin");
    rt->capturing_key = -1;
    long before = rt->launches;
    cudaGraph_t g = nullptr;
    CK(rt, cudaStreamEndCapture(rt->stream, &g));
    anvil_graph rec;
    CK(rt, cudaGraphInstantiate(&rec.exec, g, 0));
    size_t nodes = 0;
    cudaGraphGetNodes(g, nullptr, &nodes);
    cudaGraphDestroy(g);
    rec.nodes = (long)nodes;
    rec.streams_taken = rt->host_stream - rt->capture_stream0;
    rec.pending_after = rt->pending;
    rt->graphs[key] = rec;
    (void)before;
    CK(rt, cudaGraphLaunch(rec.exec, rt->stream));
    return 0;
}

// ---------------------------------------------------------------------------- device timing
static int ensure_events(anvil_rt *rt) {
    if (!rt->ev0) { CK(rt, cudaEventCreate(&rt->ev0)); CK(rt, cudaEventCreate(&rt->ev1)); }
    return 0;
}
extern "C" int anvil_rt_timer_begin(anvil_rt *rt) {
    if (ensure_events(rt)) return 1;
    CK(rt, cudaEventRecord(rt->ev0, rt->stream));
    return 0;
}
extern "C" int anvil_rt_timer_end(anvil_rt *rt, float *ms) {
    if (ensure_events(rt)) return 1;
    CK(rt, cudaEventRecord(rt->ev1, rt->stream));
    CK(rt, cudaEventSynchronize(rt->ev1));
    CK(rt, cudaEventElapsedTime(ms, rt->ev0, rt->ev1));
    return 0;
}
extern "C" int anvil_rt_time_launch(anvil_rt *rt, anvil_launch_fn launch, int index, int repeats, float *ms) {
    if (ensure_events(rt)) return 1;
    if (repeats < 1) repeats = 1;
    uint32_t stream0 = rt->host_stream, pending0 = rt->pending;
    CK(rt, cudaStreamSynchronize(rt->stream));
    CK(rt, cudaEventRecord(rt->ev0, rt->stream));
    for (int i = 0; i < repeats; i++) {
        rt->host_stream = stream0; rt->pending = pending0;      // every repeat draws the same numbers
        if (launch(rt, index)) return 1;
    }
    CK(rt, cudaEventRecord(rt->ev1, rt->stream));
    CK(rt, cudaEventSynchronize(rt->ev1));
    float total = 0;
    CK(rt, cudaEventElapsedTime(&total, rt->ev0, rt->ev1));
    *ms = total / repeats;
    return 0;
}

// ---------------------------------------------------------------------------- tensor maps
// A TMA descriptor of a row-major f32 matrix inside the arena, for the contraction templates' k-major operand feed:
// dimensions {cols, rows}, row stride in elements, box {4 columns, box_rows rows} (one 16-byte column of the operand
// tile per copy), no swizzle, zeros outside the matrix. cuTensorMapEncodeTiled is looked up through the runtime API,
// so the library does not link against the driver. Returns 0, or 1 with the reason in anvil_rt_last_error (the caller
// then launches the variant without TMA).
#include <cuda.h>
extern "C" int anvil_rt_tensor_map(anvil_rt *rt, void *map_out, size_t off, long rows, long cols, long row_stride, int box_rows) {
    typedef CUresult (*encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static encode_fn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn || q != cudaDriverEntryPointSuccess)
            return fail(rt, "anvil: cuTensorMapEncodeTiled is not available");
        encode = (encode_fn)fn;
    }
    if (in_range(rt, off, 4 * (size_t)((rows - 1) * row_stride + cols))) return 1;
    if (off % 16 || row_stride % 4 || cols % 4 || box_rows < 1 || box_rows > 256)
        return fail(rt, "anvil: operand is not 16-byte aligned for a tensor map");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_stride * 4};
    const cuuint32_t box[2] = {4, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode((CUtensorMap *)map_out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, rt->arena + off, dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(rt, "anvil: cuTensorMapEncodeTiled failed (%d)", (int)r);
    return 0;
}

// ---------------------------------------------------------------------------- collective
extern "C" void anvil_rt_set_allreduce(anvil_rt *rt, anvil_allreduce_fn fn, void *user) {
    rt->allreduce = fn;
    rt->allreduce_user = user;
}
extern "C" int anvil_rt_allreduce(anvil_rt *rt, size_t off, long count) {
    if (in_range(rt, off, 4 * (size_t)count)) return 1;
    if (!rt->allreduce) return fail(rt, "anvil: the program was sharded over several GPUs but no collective is attached");
    if (rt->capturing_key >= 0) return fail(rt, "anvil: a collective inside a recorded launch sequence");
    if (rt->allreduce(rt->allreduce_user, rt->arena + off, count, (void *)rt->stream))
        return fail(rt, "anvil: the all-reduce failed");
    return 0;
}
