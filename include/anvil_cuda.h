/* anvil_cuda.h — C ABI of libanvil_cuda.so, the B200 runtime for Anvil programs.
 *
 * The library replaces the two runtime headers that the reference pastes into every generated
 * .cu file (anvil/backend/anvil_cuda.h and anvil/backend/anvil_host.h). Where the reference keeps
 * every tensor in CUDA unified memory and synchronises the device before each host touch, this
 * runtime owns ONE cudaMalloc'd arena per context; the host never dereferences device pointers and
 * every host-side service (printing, shuffle, checkpoints, loaders) moves data with explicit copies
 * on the context's stream.
 *
 * Conventions: plain pointers and sizes only; every function that can fail returns 0 on success and
 * a non-zero status otherwise, with the text available from anvil_rt_last_error(); nothing in the
 * library calls exit(). Offsets are byte offsets into the arena. One host thread per context.
 *
 * Arena layout: bytes [0, ANVIL_RT_HEADER_BYTES) are the header (fault record, device copy of the
 * random stream counter, spare words); program buffers follow at offsets chosen by the compiler's
 * arena plan.
 */
#ifndef ANVIL_CUDA_H
#define ANVIL_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ANVIL_RT_HEADER_BYTES 256
#define ANVIL_RT_FAULT_OFF 0        /* struct { int code; int pad; long long value; }            */
#define ANVIL_RT_STREAM_OFF 16      /* uint32: device copy of the random stream counter           */
#define ANVIL_RT_STATUS_OFF 32      /* uint32: status word written by kernels that give up a wait */
#define ANVIL_RT_CHECK_OFF 48       /* uint64: smallest bad index found by the last --check scan     */
#define ANVIL_RT_TICKETS_OFF 256    /* 256 x uint32 after the header: arrival counters of split reductions that finish in
                                       their last CTA; zero between launches                                       */
#define ANVIL_RT_TICKETS 256
#define ANVIL_RT_SIDE_TICKETS_OFF 1280 /* the same again for kernels on the second stream (they run beside kernels on the first) */

typedef struct anvil_rt anvil_rt;

/* ---- context and arena ------------------------------------------------------------------------
 * Replaces the per-tensor anvil_alloc / cudaMallocManaged + memset of the reference
 * (anvil/backend/anvil_cuda.h:42-46, 82-87): one zero-filled allocation for the whole program. */
anvil_rt *anvil_rt_create(int device);
void anvil_rt_destroy(anvil_rt *rt);
int anvil_rt_arena(anvil_rt *rt, size_t bytes);
void *anvil_rt_ptr(anvil_rt *rt, size_t off);                 /* device address of an arena offset */
size_t anvil_rt_arena_bytes(anvil_rt *rt);
void *anvil_rt_stream(anvil_rt *rt);                          /* the context's cudaStream_t        */
int anvil_rt_use_stream(anvil_rt *rt, void *cuda_stream);     /* run on a caller-owned stream      */
/* Second stream (no reference counterpart: the reference launches on the default stream, anvil/backend/cuda.py:560-575).
 * fork: the launches that follow go to the second stream, after everything issued so far; back: launches go to the
 * first stream again; join: the first stream waits for the second. anvil_rt_stream() names the stream launches go to.
 * A generated program forks for kernels whose results the rest of its launch run does not need and joins at its end. */
int anvil_rt_fork(anvil_rt *rt);
int anvil_rt_back(anvil_rt *rt);
int anvil_rt_join(anvil_rt *rt);
int anvil_rt_side_stream(anvil_rt *rt, int on);                /* 0: fork becomes a no-op            */
const char *anvil_rt_last_error(anvil_rt *rt);
int anvil_rt_set_error(anvil_rt *rt, const char *message);    /* returns 1                         */

/* ---- data movement (replaces direct host access to unified memory) ---------------------------- */
int anvil_rt_h2d(anvil_rt *rt, size_t off, const void *src, size_t bytes);   /* synchronous         */
int anvil_rt_d2h(anvil_rt *rt, void *dst, size_t off, size_t bytes);         /* synchronous         */
/* From device memory owned by someone else (a `__cuda_array_interface__` argument of anvil.function; the
 * reference's pyapi has host arrays only, anvil/pyapi.py:276-296): waits for `producer_stream` (0: the device). */
int anvil_rt_d2d_async(anvil_rt *rt, size_t off, const void *src_device, size_t bytes, void *producer_stream);
int anvil_rt_h2d_async(anvil_rt *rt, size_t off, const void *pinned_src, size_t bytes);
int anvil_rt_d2h_async(anvil_rt *rt, void *pinned_dst, size_t off, size_t bytes);
/* Large copies from / to PAGEABLE host memory — the caller's own arrays behind the `anvil_input{k}` / `anvil_output{k}`
 * slots of anvil/pyapi.py:282-299: cut into 8 MiB chunks that go through two pinned buffers of the context, host threads
 * filling (draining) one while the DMA engine moves the other. h2d_staged is stream-ordered and has consumed `src` when
 * it returns; d2h_staged returns with the data in `dst`. Small copies fall through to the plain calls. */
int anvil_rt_h2d_staged(anvil_rt *rt, size_t off, const void *src, size_t bytes);
int anvil_rt_d2h_staged(anvil_rt *rt, void *dst, size_t off, size_t bytes);
int anvil_rt_zero(anvil_rt *rt, size_t off, size_t bytes);
int anvil_rt_sync(anvil_rt *rt);                              /* anvil_sync, anvil_cuda.h:55-58    */
void *anvil_rt_host_alloc(size_t bytes);                      /* pinned host memory                */
void anvil_rt_host_free(void *p);

/* ---- scalars that host control flow reads or writes ---------------------------------------------
 * Loop counters and conditions are i32/f32 0-d buffers in the arena (reference: `b[0]` on unified
 * memory, anvil/backend/cuda.py:435-456). Writes are stream-ordered kernels; reads synchronise. */
int anvil_rt_set_i32(anvil_rt *rt, size_t off, int32_t value);
int anvil_rt_set_f32(anvil_rt *rt, size_t off, float value);
int anvil_rt_add_i32(anvil_rt *rt, size_t off, int32_t delta);
int anvil_rt_read_i32(anvil_rt *rt, size_t off, int32_t *out);
int anvil_rt_read_f32(anvil_rt *rt, size_t off, float *out);

/* ---- random numbers -----------------------------------------------------------------------------
 * The counter hash of anvil/backend/anvil_host.h:17-29. A kernel that draws random numbers takes
 * the next stream number (anvil/backend/cuda.py:490-494). The host counter is authoritative; the
 * device copy in the header lets captured launch sequences be replayed: a launch passes
 * `delta = host counter - device copy` and the kernel uses `device copy + delta`. */
void anvil_rt_seed(anvil_rt *rt, uint32_t seed);              /* sets the seed, stream counter = 0 */
uint32_t anvil_rt_get_seed(anvil_rt *rt);
uint32_t anvil_rt_get_stream(anvil_rt *rt);
void anvil_rt_set_stream(anvil_rt *rt, uint32_t stream);
uint32_t anvil_rt_next_stream_delta(anvil_rt *rt);            /* takes a stream number; returns delta */
int anvil_rt_stream_commit(anvil_rt *rt);                     /* device copy += pending; delta -> 0 */
uint32_t anvil_rt_rand_bits(uint32_t idx, uint32_t stream, uint32_t salt, uint32_t seed);
float anvil_rt_rand(uint32_t idx, uint32_t stream, uint32_t salt, uint32_t seed, int open_low);

/* ---- runtime calls of the IR (anvil/backend/cuda.py:551-594; anvil_host.h:237-284) ------------ */
int anvil_rt_iota(anvil_rt *rt, size_t off, long n);
int anvil_rt_shuffle(anvil_rt *rt, size_t off, long n);       /* Fisher-Yates, anvil_host.h:269-276 */
int anvil_rt_nonzero(anvil_rt *rt, size_t src_off, long n, size_t dst_off, long size);
int anvil_rt_clock(anvil_rt *rt, size_t off);                 /* seconds since create, after a sync */
typedef struct { size_t off; uint64_t key; } anvil_rt_ckpt;  /* key: ir.ckpt_key                   */
int anvil_rt_save(anvil_rt *rt, const char *path, const anvil_rt_ckpt *tab, long n);
int anvil_rt_load(anvil_rt *rt, const char *path, const anvil_rt_ckpt *tab, long n, float *ok);
int anvil_rt_save_npy(anvil_rt *rt, const char *path, const unsigned char *header, long hlen,
                      size_t off, long bytes);
int anvil_rt_load_npy(anvil_rt *rt, const char *path, size_t off, long n, long offset, int kind, int size);
/* Data files of the other formats; the environment variable ANVIL_DATA, when set, replaces the directory of `path`
 * (anvil/backend/anvil_host.h:134-141). Errors: "anvil: cannot open data file <path>" or "anvil: data file <path>
 * does not have the shape this program was compiled for" through anvil_rt_last_error, status 1.
 *   load_idx    IDX file, plain or gzip: skip `header` bytes, n unsigned bytes -> f32 (is_int 0) or i32
 *               (anvil_host.h:143-156, anvil/interp.py:243-251)
 *   load_csv    the first n numbers after `skip` lines of a text file, any separators (anvil_host.h:179-190)
 *   load_bytes  a file of exactly n bytes, one i32 each (anvil_host.h:192-197)
 *   input       one line of standard input, its first decimal number (NaN if none) -> the f32 at `off`;
 *               *eof = 1 at the end of the input, after printing a newline (anvil_host.h:286-300) */
int anvil_rt_load_idx(anvil_rt *rt, const char *path, size_t off, long n, long header, int is_int);
int anvil_rt_load_csv(anvil_rt *rt, const char *path, size_t off, long n, long skip);
int anvil_rt_load_bytes(anvil_rt *rt, const char *path, size_t off, long n);
int anvil_rt_input(anvil_rt *rt, size_t off, int *eof);

/* ---- output (anvil_host.h:76-132) ----------------------------------------------------------------
 * Text goes to stdout/stderr, or into a capture buffer when capture is on (tests, notebooks). */
int anvil_rt_capture(anvil_rt *rt, int on);
const char *anvil_rt_captured(anvil_rt *rt);                  /* text so far; valid until next call */
int anvil_rt_print_text(anvil_rt *rt, const char *text, int to_stderr);
int anvil_rt_print_scalar(anvil_rt *rt, size_t off, int is_int, const char *fmt, int fmt_is_int, int to_stderr);
int anvil_rt_print_tensor(anvil_rt *rt, size_t off, int is_int, int rank, const long *dims);
int anvil_rt_print_pick(anvil_rt *rt, size_t off, const char *const *choices, int n, int to_stderr);
int anvil_rt_print_chars(anvil_rt *rt, size_t off, long n);
int anvil_rt_show(anvil_rt *rt, size_t off, long rows, long cols, const char *const *glyphs, int n);
int anvil_rt_flush(anvil_rt *rt);

/* ---- faults (anvil/backend/anvil_cuda.h:66-103) --------------------------------------------------
 * A failed gather bounds check inside a kernel records the first {code, value} in the header and
 * clamps the index; nothing traps. anvil_rt_check_faults synchronises, and on a fault returns 1
 * with last_error = "anvil: runtime error: <message> (got <value>)". */
int anvil_rt_fault_messages(anvil_rt *rt, const char *const *messages, int n);
int anvil_rt_check_faults(anvil_rt *rt);
int anvil_rt_oob(anvil_rt *rt, const char *message, long long value);   /* anvil_oob, anvil_host.h:69-73 */

/* ---- launch-sequence capture (no reference counterpart: the reference synchronises the device at
 * every loop iteration, anvil/backend/cuda.py:443-445). A run of kernel launches inside a loop body
 * is recorded once into a CUDA graph keyed by `key` and replayed on later iterations. */
int anvil_rt_graph_begin(anvil_rt *rt, int key);   /* 0: replayed a cached graph (skip the launches)
                                                     1: capturing now, issue the launches then _end
                                                     2: graphs are off, issue the launches, no _end
                                                    <0: error */
int anvil_rt_graph_end(anvil_rt *rt, int key);
void anvil_rt_graphs(anvil_rt *rt, int on);
/* --profile (reference: the native back end's per-kernel table, anvil/backend/aarch64.py:383-400, 921-927 and
 * runtime.s:1590-1671; `anvil run --profile`, anvil/cli.py:43). With profiling on, graphs are off, every launch
 * unit of a generated program brackets itself with prof_begin / prof_end (two CUDA events and a synchronise; no-ops
 * otherwise), and the program's main prints
 *     "\n  time%        ms      calls   kernel\n"  then  "%6.1f%%  %8.1f  %9lld   %s\n" per unit in first-run order
 *     and  "          %8.1f ms in kernels\n"
 * through profile_report before it returns. */
/* --check (reference: `anvil run --check[=inf]`, anvil/interp.py:408-423; aarch64.py:82-89, 459-481): mode 1 stops at
 * the first nan, mode 2 at the first nan or infinity, in any f32 tensor a launch unit wrote. Graphs are off. Every
 * launch unit of a generated program calls check_tensor for the tensors it wrote (a no-op when checking is off);
 * a hit gives status 1 and the message
 *     "anvil: runtime error: --check: nan in `name` at [i, j]\n  made by `label`:\n  computing (k12):  ..." */
void anvil_rt_check(anvil_rt *rt, int mode);
int anvil_rt_checking(anvil_rt *rt);
int anvil_rt_check_tensor(anvil_rt *rt, size_t off, long n, const char *name, const long *shape, int rank,
                          const char *made_by);
void anvil_rt_profile(anvil_rt *rt, int on);
int anvil_rt_prof_begin(anvil_rt *rt, int slot);
int anvil_rt_prof_end(anvil_rt *rt, int slot);
int anvil_rt_profile_report(anvil_rt *rt, const char *const *names, int n);
/* What --profile has accumulated for one launch unit so far: total milliseconds and calls; 1 if it never ran.
 * (`anvil cost --cuda` puts these beside the static estimate of anvil/cost.py:116-150.) */
int anvil_rt_profile_get(anvil_rt *rt, int slot, double *milliseconds, long *calls);
long anvil_rt_launch_count(anvil_rt *rt);          /* kernels launched (graph replays count their nodes) */
void anvil_rt_count_launches(anvil_rt *rt, long n);

/* ---- device timing (no reference counterpart; the reference's `--profile` reads a CPU counter
 * around every kernel call, anvil/backend/aarch64.py:382-402). CUDA events on the context's stream. */
int anvil_rt_timer_begin(anvil_rt *rt);
int anvil_rt_timer_end(anvil_rt *rt, float *milliseconds);    /* synchronises on the end event   */
/* Times ONE call of a program's kernel launcher (`launch(rt, index)` as exported by a generated
 * library) `repeats` times back to back and returns the mean milliseconds per call. */
typedef int (*anvil_launch_fn)(anvil_rt *, int);
int anvil_rt_time_launch(anvil_rt *rt, anvil_launch_fn launch, int index, int repeats, float *milliseconds);

/* ---- TMA descriptors for the contraction templates (no reference counterpart: its kernels read operands with plain
 * loads, anvil/backend/cuda.py:282-313). Writes a 128-byte CUtensorMap for the row-major f32 matrix of `rows` x `cols`
 * elements at arena offset `off` (rows `row_stride` elements apart; offset, stride and cols multiples of 16 bytes) with a
 * box of 4 columns x `box_rows` rows, zeros outside the matrix, into `map_out` (64-byte aligned host memory). */
int anvil_rt_tensor_map(anvil_rt *rt, void *map_out, size_t off, long rows, long cols, long row_stride, int box_rows);

/* ---- the data-parallel collective (no reference counterpart: the reference is single-device).
 * Sums `count` f32 values at arena offset `off` over all ranks, in place, stream-ordered. The
 * collective is either supplied by the host program through the callback below, or the runtime's own (next block). */
typedef int (*anvil_allreduce_fn)(void *user, void *device_ptr, long count, void *cuda_stream);
void anvil_rt_set_allreduce(anvil_rt *rt, anvil_allreduce_fn fn, void *user);
int anvil_rt_allreduce(anvil_rt *rt, size_t off, long count);
/* The collective inside the runtime: NCCL (dlopen'ed "libnccl.so.2") over NVLink / NVSwitch, so that a C host can run
 * data parallel without Python. Rank 0 makes a 128-byte id and hands it to the other ranks by whatever means the host
 * program has; every rank then joins. After anvil_rt_comm_init, anvil_rt_allreduce is ncclAllReduce(sum, f32) in place on
 * the arena, ordered on the context's stream. Algorithm, protocol and channel count are pinned (Ring / Simple / 8) unless
 * the environment sets them, for run-to-run identical sums at a given number of ranks. */
int anvil_rt_comm_unique_id(void *id_out, size_t bytes);
int anvil_rt_comm_init(anvil_rt *rt, int rank, int nranks, const void *unique_id, size_t bytes);
int anvil_rt_comm_nranks(anvil_rt *rt);            /* ranks of the communicator this context joined, 0 if none */
int anvil_rt_comm_destroy(anvil_rt *rt);

/* ---- the bounded wait of the tensor-core templates, exercised on purpose (no reference counterpart: the
 * reference's kernels never wait on one another). Runs one tiny kernel that waits, with a limit of `limit_clocks`
 * SM clocks (at most 2^31), on a barrier nothing arrives on; the kernel gives up when the limit runs out, records
 * the time-out in the arena header's status word like a contraction kernel would, and returns. `*status_out`
 * receives that word (0x7C05 after a time-out), `*waited_clocks` the clocks spent waiting. The status word stays
 * set, so the next anvil_rt_check_faults reports "a kernel gave up waiting on a barrier"; clear it with
 * anvil_rt_zero(rt, ANVIL_RT_STATUS_OFF, 4). Nothing traps and the context stays usable. */
int anvil_rt_selftest_wait(anvil_rt *rt, long long limit_clocks, uint32_t *status_out, long long *waited_clocks);

/* ---- column sums without allocation (no counterpart in the reference: its runtime allocates every
 * tensor with cudaMallocManaged and has no entry point a caller could use under a no-allocation rule).
 * out[j] = sum_i x[i * cols + j] for a row-major f32 matrix; x and out are device pointers supplied by
 * the caller, the launch goes to `cuda_stream`. It is the split column reduction the compiler emits
 * for bias gradients, with the partial sums kept in a fixed 4 MiB array inside the library instead of
 * the arena's scratch region, so the call performs no cudaMalloc / cudaFree at all. For callers that
 * must not allocate: plug-ins inside a framework that owns device memory through its own pool,
 * processes with a memory budget fixed at start-up, latency-critical loops.
 * Returns 0, 1 (bad arguments), 2 (cols x splits exceeds ANVIL_COLSUM_STATIC_MAX_PARTIALS), 3 (CUDA
 * error); the reason is printed on stderr. Every GPU that loads the library holds the array until the
 * process ends; all calls share it, so calls that overlap on the GPU race (calls on one stream are
 * ordered). The first call on a device resolves the array's address: make it outside stream capture. */
#define ANVIL_COLSUM_STATIC_MAX_PARTIALS (1 << 20)
int anvil_colsum_f32_static(const float *x, long rows, long cols, float *out, void *cuda_stream);

#ifdef __cplusplus
}
#endif
#endif
