/*
 * raf_b200 - C ABI of the B200-native ZeRO optimizer step for RAF's operator API.
 *
 * One shared library (libraf_b200.so) exports everything below with C linkage,
 * plain pointers and sizes.  A RAF dialect (an OpEnv per operator, see
 * raf_b200/csrc/raf_dialect) forwards DLTensor::data pointers to these entry
 * points; the Python mirror under raf_b200/ binds them with ctypes.
 *
 * Conventions
 *   - every function returns a rafb200_status (0 = success); the message of
 *     the last failure on the calling thread is rafb200_last_error().
 *     Nothing in this library calls exit() or abort() (the reference's
 *     NCCL_CALL does, include/raf/communicator.h:41-49).
 *   - all device work is enqueued on the cudaStream_t the caller passes
 *     (as `void*`, like the reference's OpEnv stream requests, include/raf/op.h:86-93);
 *     no call synchronises the device unless its comment says so.
 *   - step calls allocate nothing.  Objects (tensor lists, plans, communicators)
 *     allocate their small device tables when they are created, which is the
 *     moment the reference constructs an OpEnv (once per call site and shape).
 *   - parameters, momenta and second moments are fp32.  Gradients may be
 *     fp32 / fp16 / bf16; the optional parameter copy written for the
 *     all-gather may be fp32 / fp16 / bf16.
 *   - citations "file:line" refer to the awslabs/raf source tree.
 */
#ifndef RAF_B200_H_
#define RAF_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RAFB200_API __attribute__((visibility("default")))

typedef enum {
  RAFB200_OK = 0,
  RAFB200_INVALID_ARGUMENT = 1,
  RAFB200_CUDA_ERROR = 2,
  RAFB200_NCCL_ERROR = 3,
  RAFB200_TIMEOUT = 4,          /* host-side deadline (rendezvous, communicator init) */
  RAFB200_DEVICE_WAIT_EXPIRED = 5, /* a bounded wait inside a kernel gave up */
  RAFB200_UNSUPPORTED = 6,
  RAFB200_IO_ERROR = 7
} rafb200_status;

/* Element types.  The reference's DType codes for the same types are
 * kDLFloat/32, kDLFloat/16 and kDLBfloat/16 (include/raf/device.h:27-36). */
typedef enum {
  RAFB200_F32 = 0, RAFB200_F16 = 1, RAFB200_BF16 = 2,
  /* collectives only (the NCCL type map of src/op/dialect/nccl/communication_utils.h:31-48): */
  RAFB200_F64 = 3, RAFB200_I8 = 4, RAFB200_U8 = 5, RAFB200_I64 = 6
} rafb200_dtype;

RAFB200_API const char* rafb200_last_error(void);
RAFB200_API int rafb200_version(void);

/* ------------------------------------------------------------------------- */
/* Tensor lists                                                               */
/* ------------------------------------------------------------------------- */
/*
 * A tensor list is the device-resident form of the `tensor_list` argument of
 * raf.op.lans ([g..., p..., m..., v...], python/raf/optim/lans.py:267) and of
 * the per-parameter (x, dx, v) triples of raf.op.sgd.  It replaces the
 * reference's TensorListMetadata, which is rebuilt and passed by value on
 * every launch (src/op/dialect/cuda/kernels/multi_tensor_apply.cuh:20-92):
 * geometry (element counts, work items) is fixed at creation, pointers are
 * (re)bound with rafb200_tensor_list_bind.
 *
 * numel[i] may be 0.  g_dtype is the dtype of every gradient, out_dtype of
 * every optional parameter copy.
 */
typedef struct rafb200_tensor_list_s* rafb200_tensor_list_t;

RAFB200_API int rafb200_tensor_list_create(int k, const int64_t* numel, int g_dtype, int out_dtype,
                                           rafb200_tensor_list_t* list);
/* Host arrays of k device pointers each.  g, p and m are required by every
 * optimizer here (m = SGD's momentum buffer, Adam/LANS's first moment); v is
 * required by Adam and LANS and may be NULL for SGD; out may
 * be NULL (no parameter copy) or hold NULL entries.  The table is copied to
 * the device on `stream` only when a pointer changed since the last bind. */
RAFB200_API int rafb200_tensor_list_bind(rafb200_tensor_list_t list, const void* const* g,
                                         float* const* p, float* const* m, float* const* v,
                                         void* const* out, void* stream);
RAFB200_API int rafb200_tensor_list_destroy(rafb200_tensor_list_t list);
RAFB200_API int64_t rafb200_tensor_list_total_elems(rafb200_tensor_list_t list);

/* Scheduling knobs of the LANS kernel for this list (see rafb200_lans):
 * lead_elems = how far (in elements) the gradient-norm items run ahead of the
 * other items; gap_items = work items placed between a tensor's last parked item
 * and its streamed update items (0 = one per shared-memory slot of the grid);
 * max_blocks = cap on the persistent grid (0 = one block per SM), used to leave
 * SMs to a concurrent collective.  Defaults are chosen at creation; a change
 * rebuilds the work-item table (and synchronises the device first). */
RAFB200_API int rafb200_tensor_list_tune(rafb200_tensor_list_t list, int64_t lead_elems,
                                         int gap_items, int max_blocks);
/* Bound of every wait inside the LANS kernel, in milliseconds (default 2000).
 * When a wait runs out the kernel records it and returns; rafb200_lans_status
 * then reports RAFB200_DEVICE_WAIT_EXPIRED.  The reference has no in-kernel
 * waits: its passes are separate launches. */
RAFB200_API int rafb200_tensor_list_set_wait_limit(rafb200_tensor_list_t list, int limit_ms);
/* The collectives inside the update kernels, for a caller that manages symmetric memory
 * and the cross-rank barriers itself (rafb200_zero_set_fused does both for the ZeRO step; no
 * counterpart in the reference).  After this call rafb200_sgd_list / rafb200_adam /
 * rafb200_lans on the list
 *   - with reduce_scatter != 0 take the gradient of tensor i not from its bound `g` but as
 *     the SUM over ranks of the bytes at g_offset_bytes[i] (a multiple of 16; the tensor's
 *     region zero-padded to 16 bytes) inside the symmetric gradient buffer - through g_mc
 *     (multimem.ld_reduce) when it is not NULL, else rank by rank from g_peer[0..world) in
 *     a fixed order, fp32 accumulation, one rounding to the gradient dtype - and WRITE that
 *     sum to the bound `g` (16-byte aligned, padded likewise); LANS needs normalize_grad
 *     for this (its gradient-norm pass is what reads the gradients);
 *   - with all_gather != 0 store the model-dtype copy, whose bound `out` must lie inside
 *     p_peer[rank], at the same offset into every rank's buffer: through p_mc
 *     (multimem.st) when it is not NULL, else one store per rank.
 * The caller orders the ranks: every rank's gradients are in place before any rank
 * launches, and nobody reads the parameter buffers before every rank's kernel is done.
 * world <= 16.  Takes effect with the next rafb200_tensor_list_bind. */
RAFB200_API int rafb200_tensor_list_set_symmetric(rafb200_tensor_list_t list, int world, int rank,
                                                  const void* const* g_peer, const void* g_mc,
                                                  void* const* p_peer, void* p_mc,
                                                  const int64_t* g_offset_bytes, int reduce_scatter,
                                                  int all_gather);
/* Replaces the work-item table of the LANS kernel for this list by the caller's
 * (same encoding as rafb200_lans_schedule; used with and without gradient
 * normalisation), for experiments with other orders.  The caller is responsible
 * for the order's dependencies: an item that is placed before the items it waits
 * for makes the kernel give up after the wait limit.  rafb200_tensor_list_tune
 * restores the built-in order. */
RAFB200_API int rafb200_tensor_list_set_lans_items(rafb200_tensor_list_t list, const uint32_t* items,
                                                   size_t count);

/* ------------------------------------------------------------------------- */
/* Optimizer updates (shard-local)                                            */
/* ------------------------------------------------------------------------- */
/*
 * raf.op.sgd  - schema SgdArgs{x, dx, v, learning_rate, mu}
 *   (scripts/src_codegen/def_schema.py:671-677; compute python/raf/_tvm_op/sgd.py:13-33;
 *    the traced chain multiply/add/multiply/subtract of python/raf/optim/sgd.py:198-201):
 *       v1 = mu*v0 + dx ;  x1 = x0 - learning_rate*v1
 *   evaluated in fp32 without fused multiply-add, in place on x and v.
 * Fused neighbours (no counterpart inside the reference op; pass the neutral
 * value to get the reference op exactly):
 *   grad_scale   dx is multiplied by it first (1/loss_scale, 1/n after a sum
 *                reduce-scatter; replaces the `divide` of partition_gradient.cc:274-279)
 *   weight_decay dx += weight_decay*x0 (torch.optim.SGD convention; 0 = reference)
 *   dx_dtype     fp16/bf16 gradients are widened on load (the cast of sgd.py:193-195)
 *   out          receives cast(x1, out_dtype) (the cast of sgd.py:203-204 written
 *                straight into the all-gather buffer); may be NULL.
 */
RAFB200_API int rafb200_sgd(float* x, const void* dx, int dx_dtype, float* v, int64_t numel,
                            float learning_rate, float mu, float weight_decay, float grad_scale,
                            void* out, int out_dtype, void* stream);
/* The same update over a bound tensor list in ONE launch (x = p, v = m of the list). */
RAFB200_API int rafb200_sgd_list(rafb200_tensor_list_t list, float learning_rate, float mu,
                                 float weight_decay, float grad_scale, void* stream);

/*
 * raf.op.lans - schema LansArgs{tensor_list, step, learning_rate, beta1, beta2, eps,
 *   bias_correction, weight_decay, grad_averaging, mode, normalize_grad}
 *   (scripts/src_codegen/def_schema.py:678-694; host src/op/dialect/cuda/lans.cc:25-165;
 *    kernels src/op/dialect/cuda/kernels/multi_tensor_lans.cu:95-450).
 * Same argument meaning and per-element formulas.  Differences, all deliberate:
 *   - one persistent launch instead of about fifty.  A chunk of a tensor is
 *     loaded into shared memory once and its intermediate results stay on chip
 *     (in tensor memory) while the tensor-wide norms stage 2 needs are
 *     completed by the other thread blocks, so every
 *     array is read once and written once; only the part of a tensor that
 *     exceeds what the grid can hold on chip is read a second time.  Per-tensor
 *     norms are reduced warp-shuffle-then-block in the same kernel and summed
 *     across chunks in double precision (exact, hence independent of arrival
 *     order, for any realistic tensor), not in the reference's chunk/tree order;
 *     reciprocals and square roots use the approximate (<= 1 ulp) hardware
 *     forms with fused multiply-adds: p, m, v agree with the reference
 *     arithmetic to ~3e-6 relative after 10 steps, inside the 1e-5 the path
 *     allows for LANS;
 *   - `step` is a host integer, or - when step_dev is not NULL - is read on the
 *     device from a 0-d fp32 tensor as the reference schema has it, without the
 *     blocking device-to-host copy of lans.cc:97-99;
 *   - gradients may be 16-bit and grad_scale is applied on load (replaces
 *     group_cast, python/raf/optim/lans.py:261-265); g is NOT overwritten
 *     (the reference leaves update_m in it);
 *   - `out` of the list receives cast(p_new) (python/raf/optim/lans.py:289-290);
 *   - the scratch regions of different tensors never overlap (the reference's
 *     q pointers do for three or more tensors, lans.cc:116-119).
 * workspace: rafb200_lans_workspace_bytes(list) bytes of device memory owned
 * by the caller (the reference requests its workspace the same way,
 * lans.cc:66-78); contents need not be preserved between calls.
 */
RAFB200_API size_t rafb200_lans_workspace_bytes(rafb200_tensor_list_t list);
RAFB200_API int rafb200_lans(rafb200_tensor_list_t list, int step, const float* step_dev,
                             float learning_rate, float beta1, float beta2, float eps,
                             int bias_correction, float weight_decay, int grad_averaging, int mode,
                             int normalize_grad, float grad_scale, void* workspace,
                             size_t workspace_bytes, void* stream);
/* The order in which the LANS kernel hands out its work items for a list of
 * these element counts (host only, no GPU needed; for inspection and tests).
 * An item is two words: bits 31..30 of the first = kind, bits 29..0 = tensor
 * index; the second = index of the item's chunk inside the tensor.  Kinds:
 *   0  gradient norm: sum of squares of 7168 (16-bit gradients) / 4096 (fp32)
 *      elements of g;
 *   1  "streamed" stage 1 of 1024 elements: sums of squares of p, update_m,
 *      update_g only;
 *   2  "streamed" update of 1024 elements: stage 1 again, then stage 2, stores;
 *   3  "parked": stage 1 and, once the tensor's norms are final, stage 2 of 1024
 *      elements that stay on chip in between (in a cell of the SM's tensor memory
 *      or of its shared memory).
 * The items are dealt out to the blocks of the persistent grid in turn, in this
 * order; a block works through its share in order.  Kinds 1 and 3 wait for every
 * kind-0 item of their tensor (only with normalize_grad); kind 2 and the second
 * half of kind 3 wait for every kind-1 and kind-3 item of their tensor.  An item
 * only waits for items that come earlier in the order, and at most five eighths
 * of the grid's parking places (cells_total = blocks x 29 cells) ever hold
 * parked items of one tensor, so no block ever waits for a cell that an item
 * behind it holds.  The
 * reference has no such object: its six passes are separate launches
 * (multi_tensor_lans.cu:401-450).  lead_elems and gap_items as in
 * rafb200_tensor_list_tune (gap_items 0 = cells_total).
 * items may be NULL to query *count alone; capacity counts items. */
RAFB200_API int rafb200_lans_schedule(int k, const int64_t* numel, int g_dtype, int with_norm_phase,
                                      int cells_total, int64_t lead_elems, int gap_items,
                                      uint32_t* items, size_t capacity, size_t* count);
/* How that order is dealt out to a persistent grid of `grid` blocks (host only; for
 * inspection and tests): block b runs two lists, 2b (its even slots) and 2b + 1 (its odd
 * slots); list h = items[offsets[h] .. offsets[h + 1]) in the encoding above, where the
 * second word of a kind-3 item also carries, in its top 11 bits, the item's running number
 * among the kind-3 items of its list (cells are granted by these numbers).  offsets has
 * 2 * grid + 1 entries.  cells_even / cells_odd = the cells a block's even / odd list may
 * use: a list never holds more kind-3 items of one tensor than that, which is what makes
 * the kernel's waits for cells deadlock-free.  items / offsets may be NULL. */
RAFB200_API int rafb200_lans_partition(int k, const int64_t* numel, int g_dtype, int with_norm_phase,
                                       int grid, int64_t lead_elems, int gap_items, uint32_t* offsets,
                                       uint32_t* items, size_t capacity, size_t* count,
                                       int* cells_even, int* cells_odd);
/* Synchronises `stream`, then reports whether the last rafb200_lans on this
 * workspace completed (RAFB200_OK) or a bounded device wait expired.
 * norms_host (optional, 4*k floats, tensor-major) receives
 * ||g||, ||p||, ||update_m||, ||update_g|| of every tensor. */
RAFB200_API int rafb200_lans_status(rafb200_tensor_list_t list, const void* workspace,
                                    float* norms_host, void* stream);

/*
 * LANS update of ONE tensor without any device allocation, by the library or by
 * the caller.  This entry point has no counterpart in the reference, whose
 * operator always requests a workspace from the memory pool
 * (src/op/dialect/cuda/lans.cc:66-78).  It is for callers that cannot allocate
 * at the point of the call: code running while the memory pool is being torn
 * down or is exhausted, or inside a region where the allocator must stay
 * untouched.  The arithmetic, kernel and argument meaning are those of
 * rafb200_lans on a one-tensor list (p, m, v fp32, updated in place; g of
 * g_dtype; out NULL or of out_dtype); the header, control words, descriptor row
 * and work-item table that rafb200_lans keeps in its workspace and list object
 * live in a fixed device array that is part of the library image instead.
 *   - Limit: numel <= 4,194,304 (4 Mi elements, the size the 74 KB array is laid
 *     out for).  Larger tensors are refused with RAFB200_INVALID_ARGUMENT; use
 *     rafb200_lans for them.  `step` is a host integer.
 *   - The first call on each device looks up the array's device address (once,
 *     with that device current).  Make that first call during set-up, before
 *     any stream capture is begun.
 *   - All calls on one device share the one array: two calls whose work may
 *     overlap in time (different streams, different threads) race on it.  Order
 *     them on one stream, or with events.
 *   - It reports bounded-wait expiry only through the error word inside the
 *     array; synchronise the stream and compare results if that matters.
 */
RAFB200_API int rafb200_lans_tensor_static(const void* g, int g_dtype, float* p, float* m,
                                           float* v, void* out, int out_dtype, int64_t numel,
                                           int step, float learning_rate, float beta1,
                                           float beta2, float eps, int bias_correction,
                                           float weight_decay, int grad_averaging, int mode,
                                           int normalize_grad, float grad_scale, void* stream);

/*
 * Adam / AdamW.  The reference has NO Adam operator; schema modelled on
 * raf.op.lans, arithmetic = LANS stage 1 without gradient normalisation and
 * trust ratios (multi_tensor_lans.cu:281-306):
 *   mode 1: m=b1*m+(1-b1)*g; v=b2*v+(1-b2)*g*g; p -= lr*((m/bc1)/(sqrt(v/bc2)+eps) + wd*p)
 *   mode 0: g += wd*p first, no decoupled term.
 */
RAFB200_API int rafb200_adam(rafb200_tensor_list_t list, int step, const float* step_dev,
                             float learning_rate, float beta1, float beta2, float eps,
                             int bias_correction, float weight_decay, int mode, float grad_scale,
                             void* stream);

/* ------------------------------------------------------------------------- */
/* Casts and bucket packing                                                   */
/* ------------------------------------------------------------------------- */
/* raf.op.cast (src/op/declare/transform.cc:868-890): round to nearest even. */
RAFB200_API int rafb200_cast(const void* src, int src_dtype, void* dst, int dst_dtype,
                             int64_t numel, void* stream);
/* raf.op.group_cast (src/op/declare/transform.cc:892-913): k tensors, one launch. */
RAFB200_API int rafb200_group_cast(int k, const void* const* src, int src_dtype, void* const* dst,
                                   int dst_dtype, const int64_t* numel, void* stream);
/*
 * raf.op.fuse_tensor / raf.op.defuse_tensor (src/op/dialect/cuda/memory.cc:20-134):
 * concatenate k tensors into one flat buffer and back, one launch instead of
 * one cudaMemcpyAsync per tensor.  offsets[i] is the element offset of tensor
 * i inside the flat buffer; elem_size in bytes.
 */
RAFB200_API int rafb200_fuse_tensor(int k, const void* const* src, const int64_t* numel,
                                    const int64_t* offsets, int elem_size, void* flat,
                                    void* stream);
RAFB200_API int rafb200_defuse_tensor(int k, void* const* dst, const int64_t* numel,
                                      const int64_t* offsets, int elem_size, const void* flat,
                                      void* stream);

/* ------------------------------------------------------------------------- */
/* Communicator and collectives                                               */
/* ------------------------------------------------------------------------- */
/*
 * Replaces NCCLCommunicator::make (src/distributed/cuda/nccl_communicator.cc:75-161)
 * for the global communicator.  The 128-byte NCCL id travels through a file
 * store as in the reference (NCCLIdSyncHelper, :20-69; SimpleFileStore,
 * src/distributed/cuda/nccl_utils.h:209-262): rank 0 writes
 * <store_path>/<seq>, the others poll for it.  store_path NULL reads
 * $RAF_FILE_STORE_PATH and falls back to /tmp/.raf_file_store.  Unlike the
 * reference (3 s, then LOG(FATAL)) the deadline is a parameter and expiry is
 * a returned RAFB200_TIMEOUT.  world_size 1 creates a communicator without
 * NCCL whose collectives degenerate to copies (the reference's
 * VoidCommunicator, src/distributed/common/communicator.cc:96-115).
 * Sets the calling thread's current device to `device`.
 */
typedef struct rafb200_comm_s* rafb200_comm_t;

RAFB200_API int rafb200_comm_create(int world_size, int rank, int device, const char* store_path,
                                    int timeout_ms, rafb200_comm_t* comm);
/* The id exchange on its own (host only): rank 0 publishes `nbytes` of `data`
 * as <store_path>/<key> (written to a temporary name and renamed, so readers see
 * nothing or all of it); every other rank polls every 10 ms until the file
 * holds nbytes and copies it into `data`, or returns RAFB200_TIMEOUT after
 * timeout_ms - a root that never arrives is reported, not waited for forever. */
RAFB200_API int rafb200_store_exchange(int rank, const char* store_path, int key, void* data,
                                       size_t nbytes, int timeout_ms);
/* Same as rafb200_comm_create, with the id supplied by the caller (e.g.
 * broadcast by its own launcher). */
RAFB200_API int rafb200_unique_id(void* id128);
RAFB200_API int rafb200_comm_create_with_id(int world_size, int rank, int device,
                                            const void* id128, int timeout_ms,
                                            rafb200_comm_t* comm);
/* Wraps an ncclComm_t that the caller created and keeps owning (RAF's
 * NCCLCommunicatorObj::nccl_comm, include/raf/nccl_communicator.h:21-28, as an
 * OpEnv receives it from RequestDistributed, src/op/dialect/nccl/nccl.cc:329).
 * rafb200_comm_destroy on the result frees the wrapper only.  world_size 1
 * gives the copy-only communicator and ignores nccl_comm. */
RAFB200_API int rafb200_comm_adopt(void* nccl_comm, int world_size, int rank, rafb200_comm_t* comm);
RAFB200_API int rafb200_comm_destroy(rafb200_comm_t comm);
/* Device memory for collective buffers, registered with the communicator
 * (ncclMemAlloc + ncclCommRegister) so that in-place collectives on it can take
 * NCCL's zero-copy and in-switch (NVLS) paths; plain cudaMalloc for a world of
 * one, when registration is unavailable, or when RAFB200_NCCL_REGISTER=0.  The
 * reference allocates every collective buffer from its memory pool without
 * registration (src/op/dialect/nccl/nccl.cc:119-146).  Free with
 * rafb200_comm_free before rafb200_comm_destroy; allocation is a collective-
 * free, set-up-time operation. */
RAFB200_API int rafb200_comm_alloc(rafb200_comm_t comm, size_t bytes, void** ptr);
RAFB200_API int rafb200_comm_free(rafb200_comm_t comm, void* ptr);
/*
 * Sub-communicators: the `rank_list` argument of raf.op._allreduce / _allgather /
 * _reduce_scatter (def_schema.py:699-738) - a list of groups of ranks of the global
 * communicator.  Replaces Communicator::InitSubCommunicator and CommunicatorPool
 * (src/distributed/common/communicator.cc:21-84, include/raf/communicator.h:104-147):
 * the result is the communicator of the group that names this rank (rank inside the
 * group = position in it), or a world of one when no group names it, cached under
 * the rank list and owned by `comm` (do not destroy it).  group_sizes[n_groups],
 * ranks[] = the groups one after another.  n_groups 0 returns `comm` itself.  Every
 * rank of `comm` must make the same call: the groups' ids travel in one all-gather over `comm`.
 */
RAFB200_API int rafb200_comm_sub(rafb200_comm_t comm, int n_groups, const int* group_sizes,
                                 const int* ranks, rafb200_comm_t* sub);
RAFB200_API int rafb200_comm_size(rafb200_comm_t comm);
RAFB200_API int rafb200_comm_rank(rafb200_comm_t comm);
/* Polls NCCL's asynchronous error state (the reference never does). */
RAFB200_API int rafb200_comm_check(rafb200_comm_t comm);

/*
 * raf.op._allreduce / _reduce_scatter / _group_reduce_scatter / _allgather /
 * _group_allgather (schemas scripts/src_codegen/def_schema.py:699-738; NCCL
 * dialect src/op/dialect/nccl/nccl.cc:40-399).  `computation` is one of
 * "sum", "prod", "min", "max", "avg" as in nccl.cc:57-72.  Counts are in
 * elements.  dtype may be any rafb200_dtype: the six types of the reference's
 * map (communication_utils.h:31-48) and bf16, which it lacks.  `comm` may be a
 * sub-communicator from rafb200_comm_sub (the schema's rank_list).
 * reduce_scatter: recvcount elements per rank, rank r receives block r of
 * sendbuf (dim 0 split, src/op/declare/collective_comm.cc:112-158); in place
 * when recvbuf == sendbuf + rank*recvcount.  allgather: in place when
 * sendbuf == recvbuf + rank*sendcount.  The group forms issue all k
 * collectives between ncclGroupStart/End (nccl.cc:231-242, :382-390).
 */
RAFB200_API int rafb200_allreduce(rafb200_comm_t comm, const void* sendbuf, void* recvbuf,
                                  int64_t count, int dtype, const char* computation, void* stream);
RAFB200_API int rafb200_reduce_scatter(rafb200_comm_t comm, const void* sendbuf, void* recvbuf,
                                       int64_t recvcount, int dtype, const char* computation,
                                       void* stream);
RAFB200_API int rafb200_group_reduce_scatter(rafb200_comm_t comm, int k,
                                             const void* const* sendbuf, void* const* recvbuf,
                                             const int64_t* recvcount, int dtype,
                                             const char* computation, void* stream);
RAFB200_API int rafb200_allgather(rafb200_comm_t comm, const void* sendbuf, void* recvbuf,
                                  int64_t sendcount, int dtype, void* stream);
RAFB200_API int rafb200_group_allgather(rafb200_comm_t comm, int k, const void* const* sendbuf,
                                        void* const* recvbuf, const int64_t* sendcount, int dtype,
                                        void* stream);

/*
 * DistConfig (include/raf/dist_config.h:17-48): the process-wide object the
 * reference's passes read - same fields and defaults.
 */
typedef struct {
  int scheduling_param;
  int iteration;
  int enable_data_parallel;
  int zero_opt_level;
  int enable_auto_dp_profiling;
  int auto_dp_profiling_start_iter;   /* default 2 */
  int auto_dp_profiling_end_iter;     /* default 4 */
  int64_t group_bucket_size;          /* default 5,000,000,000 elements */
} rafb200_dist_config;
RAFB200_API int rafb200_dist_config_get(rafb200_dist_config* out);
RAFB200_API int rafb200_dist_config_set(const rafb200_dist_config* in);

/*
 * Streams by tag (Stream::Get(device, tag, index), src/impl/stream_pool.cc:53-98;
 * tags of include/raf/stream_pool.h: compute 1, host-to-device 2, device-to-host 3,
 * communication 4, fuse 5, defuse 6).  Created on first use, one per (device, tag,
 * index), non-blocking; the same call returns the same stream.  A caller without
 * an executor of its own takes the two streams of rafb200_zero_step from here
 * (compute: tag 1 index 0, communication: tag 4 index 0), as the Python mirror
 * does; a NULL stream argument keeps its CUDA meaning, the default stream.
 */
RAFB200_API int rafb200_stream_get(int device, int tag, int index, void** stream);
RAFB200_API int rafb200_stream_release_all(void);

/* ------------------------------------------------------------------------- */
/* ZeRO plan: shard geometry and buckets                                      */
/* ------------------------------------------------------------------------- */
/*
 * Restates what GradientPartitioner (src/pass/partition_gradient.cc:177-205,
 * :241-330) and CommGrouper (src/pass/group_allgather.cc:60-160) decide at
 * compile time, for k parameter tensors of shape (dim0[i], row_elems[i]):
 *   shard rows   = ceil(dim0/n)  (python/raf/optim/utils.py:46-47;
 *                  partition_gradient.cc:191-197), rank r owns rows
 *                  [r*shard_rows, (r+1)*shard_rows) of the zero-padded tensor;
 *   buckets      = consecutive tensors; a tensor joins the open bucket while
 *                  open_elems + numel < bucket_elems (unpadded counts,
 *                  partition_gradient.cc:289-300, group_allgather.cc:110-145);
 *                  the last bucket is always flushed.
 * Host-only: usable without a GPU.
 */
typedef struct rafb200_plan_s* rafb200_plan_t;

RAFB200_API int rafb200_plan_create(int k, const int64_t* dim0, const int64_t* row_elems,
                                    int n_ranks, int rank, int64_t bucket_elems,
                                    rafb200_plan_t* plan);
RAFB200_API int rafb200_plan_destroy(rafb200_plan_t plan);
RAFB200_API int rafb200_plan_num_buckets(rafb200_plan_t plan);
/* Per-tensor queries; arrays of k entries, any may be NULL. */
RAFB200_API int rafb200_plan_query(rafb200_plan_t plan, int64_t* shard_rows, int64_t* shard_elems,
                                   int64_t* padded_elems, int* bucket_of);
/* Totals: unpadded, padded and per-rank shard element counts. */
RAFB200_API int rafb200_plan_totals(rafb200_plan_t plan, int64_t* elems, int64_t* padded_elems,
                                    int64_t* shard_elems);

/* ------------------------------------------------------------------------- */
/* ZeRO step                                                                  */
/* ------------------------------------------------------------------------- */
/*
 * The op sequence the reference's ZeRO pass emits after backward
 * (python/raf/optim/sgd.py:186-221, lans.py:230-313 after PartitionGradient
 * and GroupAllgather), as one call:
 *   per bucket:  [pad] -> grouped reduce-scatter of the local gradients
 *                -> shard-local update (SGD-momentum / Adam / LANS) that also
 *                   writes the model-dtype parameter block in place into the
 *                   all-gather destination
 *                -> grouped all-gather of the parameter blocks [-> slice]
 * with the collectives on `comm_stream`, the updates on `compute_stream`, and
 * events between them so that bucket b+1's reduce-scatter and bucket b-1's
 * all-gather overlap bucket b's update (the discipline EnforceSync encodes,
 * src/pass/enforce_sync.cc:45-68: compute stream 1, communication stream 4).
 *
 * Buffers (all device memory owned by the caller, k entries each):
 *   grads[i]   local gradient of tensor i, dim0 x row_elems, g_dtype; read only.
 *   params[i]  full model parameter, dim0 x row_elems, param_dtype: receives
 *              the all-gathered update.
 *   p/m/v[i]   fp32 master shard and optimizer state, shard_elems[i] each.
 * Binding is a set-up operation: when a pointer differs from the previous
 * bind it synchronises the device and rebuilds the device tables (it returns at
 * once when nothing changed).  Bind once and let backward write into the bound
 * gradient tensors; do not re-bind inside a timed step loop.
 * With more than one rank the state object owns two rank-major flat buffers per
 * bucket (gradients, parameter copies; padded elements x dtype size each in
 * total).  A step is, per bucket: one pack kernel (row block r of every gradient
 * into slot r; the zero rows of raf.op.pad are never written and stay zero),
 * ONE in-place ncclReduceScatter, the update kernel on slot `rank` (it writes
 * the parameter copy into the gather buffer), ONE in-place ncclAllGather, one
 * unpack kernel into params[i] (the strided_slice that drops the padding).  The
 * reference issues one collective per tensor inside a group
 * (src/op/dialect/nccl/nccl.cc:231-242,382-390).  Buckets are software-pipelined:
 * bucket b+1 is on the wire while bucket b is updated.
 */
typedef enum { RAFB200_OPT_SGD = 0, RAFB200_OPT_ADAM = 1, RAFB200_OPT_LANS = 2 } rafb200_optimizer;

typedef struct {
  int optimizer;        /* rafb200_optimizer */
  float learning_rate;
  float mu;             /* SGD momentum */
  float beta1, beta2, eps;
  float weight_decay;
  int bias_correction;  /* Adam / LANS */
  int grad_averaging;   /* LANS */
  int mode;             /* Adam / LANS: 0 = L2, 1 = decoupled */
  int normalize_grad;   /* LANS */
  float grad_scale;     /* extra gradient scale (1/loss_scale); the 1/n of a mean is added internally */
  int average;          /* 1: gradients are averaged over ranks ("avg"), 0: summed */
} rafb200_hyper;

/* ------------------------------------------------------------------------- */
/* Symmetric memory (no counterpart in the reference)                          */
/* ------------------------------------------------------------------------- */
/*
 * Device memory that every rank of ONE node has mapped, for the collectives this
 * library runs with its own kernels (rafb200_zero_attach_symmetric).  Each rank
 * allocates `bytes` (rounded up to the driver's granularity) with a shareable
 * handle, the ranks exchange the handles over abstract unix sockets named after
 * `key` (any string that is the same on every rank of the job and different
 * between jobs on the machine, e.g. "<master address>:<port>") and map each
 * other's memory; with want_multicast != 0, on GPUs that support it, rank 0 also
 * creates an NVSwitch multicast object that every rank binds its memory to.
 * Collective: every rank calls it, in the same order if it is called more than
 * once; a rank that does not arrive costs the others `timeout_ms`, after which
 * they get RAFB200_TIMEOUT and nothing stays allocated.  The memory is zero-
 * filled by the caller, not here.  rafb200_symm_pointers: peer[q] = rank q's
 * memory as addressable from this process (peer[rank] = this rank's own), and
 * the multicast address or NULL.  rafb200_symm_free synchronises the device and
 * unmaps everything; every rank frees, after the last kernel that used the
 * peers' memory has finished everywhere.
 */
typedef struct rafb200_symm_s* rafb200_symm_t;
RAFB200_API int rafb200_symm_alloc(int world_size, int rank, int device, size_t bytes, const char* key,
                                   int want_multicast, int timeout_ms, rafb200_symm_t* symm);
RAFB200_API size_t rafb200_symm_bytes(rafb200_symm_t symm);
RAFB200_API int rafb200_symm_pointers(rafb200_symm_t symm, void** peer, void** multicast);
RAFB200_API int rafb200_symm_free(rafb200_symm_t symm);

typedef struct rafb200_zero_s* rafb200_zero_t;

RAFB200_API int rafb200_zero_create(rafb200_plan_t plan, rafb200_comm_t comm, int g_dtype,
                                    int param_dtype, int optimizer, rafb200_zero_t* zero);
RAFB200_API int rafb200_zero_destroy(rafb200_zero_t zero);
RAFB200_API int rafb200_zero_bind(rafb200_zero_t zero, void* const* grads, void* const* params,
                                  float* const* p, float* const* m, float* const* v);
/* Enqueues one step; returns without waiting.  On return of the call the
 * compute stream has been made to wait for the last all-gather. */
RAFB200_API int rafb200_zero_step(rafb200_zero_t zero, const rafb200_hyper* hyper, int step,
                                  void* compute_stream, void* comm_stream);
/* Kernel launches and NCCL calls one step enqueues (for accounting). */
/*
 * Symmetric-memory mode (no counterpart in the reference, which always goes
 * through NCCL).  The caller provides, for the two flat bucket buffers and a
 * small signal pad, memory that EVERY rank has mapped: peer[q] is rank q's
 * buffer as addressable from this process (peer[rank] is the local one), and
 * mc is the NVSwitch multicast address bound to all of them, or NULL.  Sizes
 * come from rafb200_zero_flat_bytes; all three must be zero-filled, on every
 * rank, before the first step (the caller synchronises the ranks once after
 * clearing them).  After attaching, a step runs this library's own kernels for
 * the collectives instead of NCCL: reduce-scatter = multimem.ld_reduce of this
 * rank's slot (sum accumulated in fp32, rounded once), all-gather =
 * multimem.st of this rank's slot, on two streams so that they use the links
 * in opposite directions at the same time; without a multicast address the
 * same kernels read / write the peers one by one.  Ranks meet at two flag
 * barriers per bucket whose waits are bounded (10 s unless changed with
 * rafb200_zero_set_wait_limit).  When a wait runs out the kernel records it in
 * host-mapped memory: the next rafb200_zero_step / rafb200_zero_step_host on that
 * rank queues nothing and returns RAFB200_DEVICE_WAIT_EXPIRED (no device
 * synchronisation needed), and so does rafb200_zero_status after synchronising.
 * The ranks are then out of step (the late rank's barrier epochs lag): destroy
 * the state on every rank and create it again; results of the step that timed
 * out are invalid.  comm_blocks = thread blocks per collective kernel
 * (0 = default: 128 with a multicast address, four per SM without).
 * How the memory is obtained is the caller's business (cuMemCreate +
 * cuMulticastBindMem, or torch.distributed._symmetric_memory as the Python
 * layer of this package does).  Call between rafb200_zero_create and
 * rafb200_zero_bind, on every rank or on none.
 */
/*
 * The collectives INSIDE the update kernel (symmetric mode only; no counterpart
 * in the reference, whose collectives are separate NCCL launches, nccl.cc:189-190,308,387).
 * LANS, mode 1: the kernel's gradient-norm items read the sum over ranks of their chunk through
 * the switch (multimem.ld_reduce, or the peers one by one without a multicast address), write
 * it to the local gradient block for the later stages and square what they wrote; the
 * reduce-scatter kernels disappear.  mode 2: in addition stage 2 stores the model-dtype copy
 * into every rank's parameter buffer (multimem.st, or peer stores); the all-gather kernels
 * disappear too.  A step is then: pack (tensors bound outside the buffer) -> one barrier ->
 * ONE update launch over all tensors -> one barrier -> unpack, on the compute stream; link
 * traffic and memory traffic interleave inside the kernel instead of running as separate
 * kernels.  SGD and Adam do the same in their single pass (mode 1: the gradient is read as
 * the sum over ranks; mode 2: the copy is stored everywhere too).  LANS needs normalize_grad
 * (the gradient-norm pass is what reads the gradients); a LANS step without it, and every step
 * of the host-buffer form, takes the bucketed pipeline.  mode 3 = mode 2 with the copies going
 * out as one store per peer even when a multicast address exists (the better choice on two
 * ranks, where the switch would also carry the rank's own half).  Call after rafb200_zero_attach_symmetric and
 * before rafb200_zero_bind, with the same mode on every rank.
 */
RAFB200_API int rafb200_zero_set_fused(rafb200_zero_t zero, int mode);
RAFB200_API int rafb200_zero_flat_bytes(rafb200_zero_t zero, size_t* g_bytes, size_t* p_bytes,
                                        size_t* signal_bytes);
RAFB200_API int rafb200_zero_attach_symmetric(rafb200_zero_t zero, void* const* g_peer, void* g_mc,
                                              void* const* p_peer, void* p_mc,
                                              void* const* signal_peer, int comm_blocks);
/* Symmetric mode lays each flat buffer out tensor by tensor: tensor i owns n
 * row blocks of align8(shard_elems[i]) elements, starting elem_offset[i]
 * elements into the buffer (the same offset in the gradient and in the
 * parameter buffer).  Where natural[i] is 1 (shard size a multiple of 8
 * elements) that region IS the zero-padded tensor in its ordinary row-major
 * layout, so the caller may keep its gradient and / or model parameter there:
 * rafb200_zero_bind recognises grads[i] == g_peer[rank] + elem_offset[i] *
 * sizeof(g dtype) (params[i] likewise) and then skips the pack (unpack) copy of
 * that tensor - gradients are reduced from where backward wrote them and the
 * gathered parameters land where the model reads them.  The gradients are not
 * modified (sums go to a shard-sized buffer of the step object). */
RAFB200_API int rafb200_zero_arena_offsets(rafb200_zero_t zero, int64_t* elem_offset, int* natural);
RAFB200_API int rafb200_zero_status(rafb200_zero_t zero);
/* Bound of every cross-GPU wait of the symmetric mode, in milliseconds (default
 * 10000).  A rank may legitimately be late by a data-loader stall or a checkpoint:
 * choose the limit above the longest skew the job tolerates.  The reference has no
 * such limit: a rank that never joins a collective hangs the job
 * (src/op/dialect/nccl/nccl.cc:308,387 enqueue and never look back). */
RAFB200_API int rafb200_zero_set_wait_limit(rafb200_zero_t zero, int limit_ms);
/* Device address of the gradient block the update of tensor `tensor` reads: the
 * caller's gradient with one rank, this rank's reduced row block (the output of
 * the reduce-scatter, valid once a step's reduce-scatter of that bucket is
 * complete) otherwise.  shard_elems[tensor] elements of the gradient dtype.  It is
 * what the sliced `dxi` of python/raf/optim/lans.py:254-259 holds. */
RAFB200_API int rafb200_zero_shard_grad(rafb200_zero_t zero, int tensor, const void** ptr);
/* Measurement aid: issue only the selected stages of a multi-rank step
 * (bit 0 pack, 1 reduce-scatter, 2 update, 3 all-gather, 4 unpack; default 31).
 * With a stage missing the results are meaningless; every rank must use the
 * same mask.  bench.py uses it to time the stages separately. */
RAFB200_API int rafb200_zero_set_stage_mask(rafb200_zero_t zero, int mask);
/* Per step: kernels of this library (update, pack, unpack and, in symmetric mode,
 * the collective and barrier kernels) and NCCL calls (0 in symmetric mode). */
RAFB200_API int rafb200_zero_launch_counts(rafb200_zero_t zero, int* kernels, int* collectives);
/* Cap on the persistent update grids while collectives are in flight (0 = no cap). */
RAFB200_API int rafb200_zero_set_update_blocks(rafb200_zero_t zero, int max_blocks);

/* ------------------------------------------------------------------------- */
/* Host-buffer convenience: one optimizer step with the gradients in host      */
/* memory and the updated model-dtype parameters read back, the form a         */
/* caller without device buffers (a CPU executor) would use.  Copies run on    */
/* `stream`; pinned host memory makes them asynchronous.                       */
/* ------------------------------------------------------------------------- */
/* The call enqueues and returns; `compute_stream` ends up waiting for the last  */
/* copy to the host.  One cudaMemcpyAsync per tensor and direction, unless the   */
/* caller declared arenas (below).                                               */
RAFB200_API int rafb200_zero_step_host(rafb200_zero_t zero, const rafb200_hyper* hyper, int step,
                                       const void* const* grads_host, void* const* params_host,
                                       void* compute_stream, void* comm_stream);
/* Declares [base, base + bytes) - host or device memory - to be ONE allocation.
 * rafb200_zero_step_host merges the copies of tensors that follow one another
 * without a gap on both sides when source and destination each lie inside one
 * declared range: a caller that keeps its host gradients in one pinned arena, its
 * host parameters in another and the bound device tensors likewise pays one copy
 * per bucket and direction instead of one per tensor (782 for BERT-large).
 * Undeclared memory is never merged, because a copy may not span two allocations. */
RAFB200_API int rafb200_zero_declare_arena(rafb200_zero_t zero, const void* base, size_t bytes);
/* What rafb200_zero_step_host copies back: 0 (default) the whole of every
 * parameter on every rank; 1 only the rows this rank owns (rows
 * [rank*shard_rows, (rank+1)*shard_rows) of each tensor, written at the same
 * offset of params_host[i]), so that n ranks sharing one host move each
 * parameter across PCIe once, not n times. */
RAFB200_API int rafb200_zero_set_host_output(rafb200_zero_t zero, int mode);

#ifdef __cplusplus
}
#endif
#endif /* RAF_B200_H_ */
