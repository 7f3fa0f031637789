/*
 * minuet_b200 -- C ABI of the B200-native sparse-convolution hot path.
 *
 * One shared library (libminuet_b200.so), plain pointers and sizes, no torch
 * types.  Every entry point that touches the GPU only ENQUEUES work on the
 * caller's stream and returns; it never allocates, frees or synchronises, and
 * keeps no pointer after it returns.  Outputs and scratch ("workspace") are
 * allocated by the caller.  Host-side planners are pure functions.
 *
 * Every function returns an mn_status; on failure mn_last_error() gives a
 * thread-local message.  Each declaration cites the entry of the reference's
 * pybind11 module (minuet.nn.functional._C) that it stands in for.
 *
 * Conventions
 *   coordinates  int32 [n, ndim] row-major, ndim in 1..4, sorted cloud-major
 *                then lexicographically (dimension 0 most significant)
 *   batch_dims   int64 [num_clouds + 1] device prefix offsets, or NULL for one
 *                cloud (num_clouds is then ignored)
 *   kernel map   int32 [O, T] row-major; -1 marks "no source"
 *   masks        int32 [O, S] and [O, T]
 *   stream       a cudaStream_t passed as void*
 */
#ifndef MINUET_B200_H_
#define MINUET_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  MN_OK = 0,
  MN_ERR_BAD_ARG = 1,     /* shape / pointer / range check failed            */
  MN_ERR_UNSUPPORTED = 2, /* legal in the reference, not implemented here    */
  MN_ERR_WORKSPACE = 3,   /* workspace smaller than mn_*_workspace_bytes     */
  MN_ERR_CUDA = 4,        /* a CUDA runtime call or launch failed            */
  MN_ERR_DEVICE = 5       /* a kernel reported a bounded-wait timeout        */
} mn_status;

typedef enum { MN_F32 = 0, MN_F16 = 1, MN_BF16 = 2 } mn_dtype;

#define MN_MAX_NDIM 4
#define MN_MAX_OFFSETS 128

/* Control block: MN_CTRL_WORDS int32 words of DEVICE memory (256-byte aligned)
 * that the caller zeroes once and then keeps for as long as it uses the library
 * on that stream.  Word MN_CTRL_STATUS collects MN_STATUS_* bits raised by
 * kernels; the rest is the state of the grid-wide barrier that the cooperative
 * kernels (key build, radix sort, unique, mask emission) share: an arrival
 * counter on a cache line of its own and MN_CTRL_GEN_COPIES copies of the
 * generation word, 128 bytes apart, so that the polling blocks spread over
 * several L2 lines instead of queueing behind the arrivals.  The barrier state
 * is back to its idle value whenever no kernel is in flight.  Every parameter
 * called `ctrl` or `status_dev` below points at such a block.  Calls whose
 * kernels may overlap on the GPU (different streams) need a block each. */
#define MN_CTRL_WORDS 1024
#define MN_CTRL_STATUS 0
#define MN_CTRL_BARRIER_COUNT 32      /* byte offset 128 */
#define MN_CTRL_BARRIER_GEN 64        /* copy k at word MN_CTRL_BARRIER_GEN + 32 * k */
#define MN_CTRL_GEN_COPIES 16

#define MN_STATUS_KEY_BOX 2       /* a coordinate fell outside the key box              */
#define MN_STATUS_TC_TIMEOUT 4    /* a bounded barrier wait of a tensor-core kernel ran out */
#define MN_STATUS_KEY_BITS 8      /* the bounding box needs more than 63 key bits       */
#define MN_STATUS_GRID_TIMEOUT 16 /* a bounded grid-barrier wait ran out                 */

/* How coordinates are packed into one 64-bit sort/search key:
 * key = cloud << cloud_shift | sum_k (c[k] - base[k]) << shift[k].
 * A plain struct; pass it by pointer (host memory).  Two ways to obtain one:
 * mn_keyspec_make fills every field on the host from a bounding box that was
 * read back; mn_keyspec_device derives the layout ON the device and leaves it
 * there (no read-back): the host struct then only carries ndim, margin and
 * device_copy, and every kernel reads the field layout through device_copy. */
typedef struct {
  int32_t ndim;
  int32_t total_bits;       /* bits used by the key, <= 63                    */
  int32_t margin;           /* offsets up to +-margin never leave a field     */
  int32_t cloud_shift;
  int32_t cloud_bits;
  int32_t shift[MN_MAX_NDIM];
  int32_t bits[MN_MAX_NDIM];
  int64_t base[MN_MAX_NDIM];   /* coordinate that maps to field value 0       */
  int64_t extent[MN_MAX_NDIM]; /* largest legal field value                   */
  const void *device_copy;     /* NULL, or a device mn_keyspec that overrides the layout above */
} mn_keyspec;

/* Version of this interface; mn_version() returns the value the library was
 * built with.  A binding should refuse a library whose version differs from the
 * header it was written against: argument lists change between versions. */
#define MN_ABI_VERSION 14

const char *mn_last_error(void);
int mn_version(void);

/* Instrumentation (no counterpart in the reference, which only times whole
 * stages in TimeGather/TimeGEMM/TimeScatter): number of kernels this library
 * has launched so far; and, while enabled, a CUDA-event pair around every
 * launch.  mn_profile_report waits for the recorded events, writes one text
 * line "kernel launches total_ms" per kernel name into buf, clears the record
 * and returns the bytes written.  Profiling creates events, so keep it off
 * inside timed regions and stream captures. */
long long mn_launch_count(void);
void mn_profile_enable(int on);
int mn_profile_report(char *buf, int buf_bytes);

/* ---- Map step ------------------------------------------------------------ */

/* Bounding box of up to two coordinate arrays (b may be NULL):
 * minmax_dev[0..3] = per-dimension min, [4..7] = max (int32, device).
 * Stands in for GetCoordinatesMinMax, the first step of
 * _C.cuda_arg_sort_coordinates (csrc/minuet/cuda/functions/arg_sort_coodrinates.cu:31-85). */
mn_status mn_bbox(const int32_t *a, int64_t na, const int32_t *b, int64_t nb,
                  int ndim, int32_t *minmax_dev, void *ws, size_t ws_bytes,
                  void *stream);

/* Host: derive the key layout from a bounding box (host copy of mn_bbox's
 * output), the number of clouds and the largest |offset| that will be added to
 * a coordinate.  Plays the role of IsFlattenable + the flattening strides
 * (arg_sort_coodrinates.cu:220-244, kernels/flatten_coordinates.cuh:23-38).
 * MN_ERR_UNSUPPORTED when the box does not fit 63 bits. */
mn_status mn_keyspec_make(const int32_t *minmax_host, int ndim,
                          int64_t num_clouds, int32_t margin, mn_keyspec *spec);

/* Bounding box, key layout and (when keys_out != NULL) the keys of the same rows
 * in one launch, entirely on the device: the layout is written to spec_dev
 * (device memory, at least sizeof(mn_keyspec) bytes, 16-byte aligned, owned by
 * the caller for as long as keys built from it are in use) and never read
 * back; *spec (host) is filled with ndim, margin and device_copy = spec_dev and
 * can be passed wherever a key spec is expected.  A box that needs more than 63
 * key bits raises MN_STATUS_KEY_BITS in the status word.  Same role as mn_bbox +
 * mn_keyspec_make + mn_pack_keys without the device-to-host read between them
 * (the reference blocks on that read, arg_sort_coodrinates.cu:286-287).
 * ctrl: the control block. */
mn_status mn_keyspec_device(const int32_t *coords, int64_t n, int ndim,
                            const int64_t *batch_dims, int64_t num_clouds,
                            int32_t margin, void *spec_dev, mn_keyspec *spec,
                            uint64_t *keys_out, int32_t *ctrl, void *ws, size_t ws_bytes,
                            void *stream);

/* Pack coordinates into keys.  tstride (host, may be NULL) floors every
 * coordinate to a multiple of tstride[k] first, as
 * KernelMapCache.get_target_coordinates does (minuet/nn/convolutions.py:85-87).
 * status_dev (int32, device, caller-zeroed) gets bit 1 set when a coordinate
 * falls outside the spec's box. */
mn_status mn_pack_keys(const int32_t *coords, int64_t n, int ndim,
                       const int64_t *batch_dims, int64_t num_clouds,
                       const int32_t *tstride, const mn_keyspec *spec,
                       uint64_t *keys_out, int32_t *status_dev, void *stream);

/* _C.cuda_arg_sort_coordinates / _C.cuda_multi_arg_sort_coordinates
 * (csrc/minuet/torch/cuda_arg_sort_coordinates.cu:8-66): stable arg-sort,
 * cloud-major then lexicographic.  index_out int64 [n]. */
mn_status mn_arg_sort_coordinates(const int32_t *coords, int64_t n, int ndim,
                                  const int64_t *batch_dims, int64_t num_clouds,
                                  const mn_keyspec *spec, int64_t *index_out,
                                  int32_t *status_dev, void *ws, size_t ws_bytes,
                                  void *stream);

/* The same permutation without a packed key: one stable radix sort per dimension, last
 * dimension first, then one on the cloud (the reference's fallback for boxes whose
 * flattened range exceeds 64 bits and its enable_flattening = False path,
 * arg_sort_coodrinates.cu:333-359, 454-468).  Any int32 coordinates; needs no bounding
 * box and no key layout.  ctrl: the caller's control block (MN_CTRL_WORDS words);
 * workspace: mn_map_workspace_bytes(n, n, 1). */
mn_status mn_arg_sort_coordinates_by_dimension(const int32_t *coords, int64_t n, int ndim,
                                               const int64_t *batch_dims, int64_t num_clouds,
                                               int64_t *index_out, int32_t *ctrl, void *ws,
                                               size_t ws_bytes, void *stream);

/* _C.cuda_unique_coordinates / _C.cuda_multi_unique_coordinates
 * (csrc/minuet/torch/cuda_unique_coordinates.cu:8-81) on SORTED coordinates:
 * indices_out int64 [n+1] (indices[i+1] = #unique among rows 0..i),
 * unique_out int32 [n, ndim] (first indices[n] rows valid). */
mn_status mn_unique_coordinates(const int32_t *coords, int64_t n, int ndim,
                                const int64_t *batch_dims, int64_t num_clouds,
                                int32_t *unique_out, int64_t *indices_out,
                                void *ws, size_t ws_bytes, void *stream);

/* Same result as mn_unique_coordinates for callers that cannot hand over a
 * workspace because they are not allowed to allocate device memory where this
 * runs (inside a stream capture, under an allocator-free hot loop, or in a
 * plugin with a fixed memory budget).  It has no counterpart in the reference.
 * The scratch (block counts) is a fixed array inside the library image, about
 * 33 KB on every GPU that loads the library, which bounds one call to
 * 16 777 216 rows; larger n returns MN_ERR_BAD_ARG with a message that names
 * the limit.  It calls no cudaMalloc/cudaFree or allocating library routine.
 * The first call on each device looks up the array's device address (the
 * device that owns the pointers must be current); make that first call before
 * any stream capture begins.  All calls share the one array: calls whose
 * kernels can overlap on the GPU (different streams, or different host threads
 * on one device) race and must be serialised by the caller.  Nothing in the
 * array has to start at zero; each call writes every word before reading it. */
mn_status mn_unique_coordinates_static(const int32_t *coords, int64_t n, int ndim,
                                       const int64_t *batch_dims, int64_t num_clouds,
                                       int32_t *unique_out, int64_t *indices_out,
                                       void *stream);

/* Fused target-coordinate build of a strided convolution
 * (KernelMapCache.get_target_coordinates, minuet/nn/convolutions.py:85-96):
 * floor to the target stride, sort, unique; two launches.  Outputs: unique_out
 * int32 [n, ndim], keys_out uint64 [n] (sorted unique keys), and meta_out int64
 * [num_clouds + 3] = { number of unique rows, batch_dims of the result
 * [num_clouds + 1], copy of the status word }, so that one small read brings
 * back everything the host needs.  batch_dims == NULL means one cloud
 * (meta_out then has 4 entries).  ctrl: the control block. */
mn_status mn_downsample_coordinates(const int32_t *coords, int64_t n, int ndim,
                                    const int64_t *batch_dims, int64_t num_clouds,
                                    const int32_t *tstride, const mn_keyspec *spec,
                                    int32_t *unique_out, uint64_t *keys_out,
                                    int64_t *meta_out, int32_t *ctrl, void *ws,
                                    size_t ws_bytes, void *stream);

/* _C.cuda_query_sorted_index_with_offsets / _C.cuda_multi_query_...
 * (csrc/minuet/torch/cuda_sparse_convolution_mapping.cu:9-100) on packed keys:
 * kernel_map[o, t] = s with source_keys[s] == target_keys[t] + offsets[o].
 * offsets is a HOST array int32 [O, ndim]. */
mn_status mn_query_sorted_index_with_offsets(const uint64_t *source_keys, int64_t S,
                                             const uint64_t *target_keys, int64_t T,
                                             const int32_t *offsets, int64_t O,
                                             const mn_keyspec *spec,
                                             int32_t *kernel_map_out, void *stream);

/* _C.cuda_compute_kernel_map_sizes (cuda_sparse_convolution_mapping.cu:102-125). */
mn_status mn_compute_kernel_map_sizes(const int32_t *kernel_map, int64_t O, int64_t T,
                                      int32_t *sizes_out, void *stream);

/* _C.cuda_compute_kernel_map_masks (cuda_sparse_convolution_mapping.cu:127-155). */
mn_status mn_compute_kernel_map_masks(const int32_t *kernel_map, int64_t O, int64_t S,
                                      int64_t T, int32_t *source_masks_out,
                                      int32_t *target_masks_out, void *ws,
                                      size_t ws_bytes, void *stream);

/* Fused KernelMapCache.get_kernel_map (minuet/nn/convolutions.py:149-170):
 * query + sizes + stable ascending size order + both masks without ever
 * materialising the [O, T] kernel map.  target_keys == source_keys (same
 * pointer) selects the submanifold shortcut.  order_out int32 [O]
 * (order[p] = offset index at mask row p; identity when reorder == 0),
 * sizes_out int32 [O + 1]: sizes of the mask rows (i.e. sorted), followed by a
 * copy of the status word taken when the masks were written, so that one
 * device-to-host copy brings back both.  source_bits_out uint32 [S] and
 * target_bits_out uint32 [T] (each may be NULL) receive one word per row whose
 * bit p is set when mask row p has an entry for that row: the forward kernels
 * walk a row's pairs through these words instead of scanning O mask rows.
 * ctrl: the control block. */
mn_status mn_build_kernel_map(const uint64_t *source_keys, int64_t S,
                              const uint64_t *target_keys, int64_t T,
                              const int32_t *offsets, int64_t O,
                              const mn_keyspec *spec, int reorder,
                              int32_t *source_masks_out, int32_t *target_masks_out,
                              int32_t *order_out, int32_t *sizes_out,
                              uint32_t *source_bits_out, uint32_t *target_bits_out,
                              int32_t *ctrl, void *ws, size_t ws_bytes, void *stream);

/* Upper bound of the workspace any Map-step entry point needs. */
size_t mn_map_workspace_bytes(int64_t S, int64_t T, int64_t O);

/* ---- Gather - grouped GEMM - Scatter ------------------------------------- */

/* Host: GeneratePaddingBuckets + ComputeCumsumKernelPaddedSizes
 * (csrc/minuet/cuda/functions/sparse_convolution.cu:17-43, 273-292).
 * has_threshold == 0 means threshold None.  buckets_out int64 [O+1],
 * cumsum_out int64 [O+1]; *num_buckets_out = number of buckets. */
mn_status mn_plan_buckets(const int32_t *sizes, int64_t O, int has_threshold,
                          double threshold, int64_t *buckets_out,
                          int64_t *cumsum_out, int64_t *num_buckets_out);

/* Workspace of mn_sparse_convolution_forward for host-known sorted sizes. */
size_t mn_conv_workspace_bytes(const int32_t *sizes_host, int64_t O, int64_t S,
                               int64_t T, int64_t c_in, int64_t c_out,
                               mn_dtype dtype, int allow_shortcut,
                               int has_threshold, double threshold);

/* _C.cuda_sparse_convolution_forward
 * (csrc/minuet/torch/cuda_sparse_convolution_forward.cu:136-213).
 * sizes_host: HOST copy of the mask-row sizes; order: DEVICE int32 [O] or NULL.
 * status_dev: DEVICE int32 word (may be NULL, which keeps fp16/bf16 on the SIMT
 * GEMM); the tensor-core GEMM sets bit 2 there if one of its bounded barrier
 * waits expires instead of hanging. */
mn_status mn_sparse_convolution_forward(
    int64_t S, int64_t T, int64_t O, int64_t c_in, int64_t c_out, mn_dtype dtype,
    const void *sources, const void *weights, const int32_t *source_masks,
    const int32_t *target_masks, const int32_t *order, const int32_t *sizes_host,
    int gather_tile, int scatter_tile, int allow_shortcut, int has_threshold,
    double threshold, void *targets_out, int32_t *status_dev, void *ws, size_t ws_bytes,
    void *stream);

/* _C.cuda_time_gather / cuda_time_scatter / cuda_time_gemm
 * (cuda_sparse_convolution_forward.cu:8-134): enqueue only the named stage of
 * the forward pass on the workspace (contents unspecified), so the caller can
 * bracket it with events.  stage: 0 gather, 1 gemm, 2 scatter. */
mn_status mn_conv_stage(int stage, int64_t S, int64_t T, int64_t O, int64_t c_in,
                        int64_t c_out, mn_dtype dtype, const void *sources,
                        const void *weights, const int32_t *source_masks,
                        const int32_t *target_masks, const int32_t *order,
                        const int32_t *sizes_host, int tile, int allow_shortcut,
                        int has_threshold, double threshold, void *targets_out,
                        int32_t *status_dev, void *ws, size_t ws_bytes, void *stream);

/* ---- Fused (implicit-GEMM) forward ----------------------------------------- */
/* No single counterpart in the reference: replaces the gather + bucket GEMMs +
 * scatter + centre GEMM sequence of SparseConvolutionForward
 * (csrc/minuet/cuda/functions/sparse_convolution.cu:505-661) by one kernel that
 * keeps a 128-row target tile in TMEM and accumulates every offset into it.
 * fp16/bf16, at most 32 offsets, channels multiple of 8, c_out <= 256. */
int mn_implicit_supported(int64_t O, int64_t c_in, int64_t c_out, mn_dtype dtype);

/* Neighbour table of a kernel map given as masks: nbr_out int32 [O, T] holds the
 * source row feeding target t under mask row p, or -1; tile_bits_out uint32
 * [ceil(T/128)] has bit p set when any target of that 128-row tile has a
 * source under mask row p.  sizes_host: HOST sizes of the mask rows. */
size_t mn_neighbor_table_workspace_bytes(const int32_t *sizes_host, int64_t O, int64_t T);
/* With perm_out (int32 [T]) the rows of the table are a permutation of the targets:
 * perm_out[r] is the target row at table position r, chosen so that targets with the
 * same set of offsets (equal hit words, target_bits as written by mn_build_kernel_map;
 * stable sort on the Gray-sequence rank of the bit-reversed word) sit in the same 128-row tiles and tiles can skip the offsets none of their rows has.
 * nbr_out and tile_bits_out are then in table order; the forward pass takes perm and
 * writes every output row at its own place.  perm_out NULL: table order = target order
 * (ctrl is then not read).  source_bits / target_bits (each may be NULL) let the build
 * read only the mask entries that hold a pair instead of whole mask rows. */
mn_status mn_build_neighbor_table(const int32_t *source_masks, const int32_t *target_masks,
                                  const int32_t *sizes_host, int64_t O, int64_t S, int64_t T,
                                  const uint32_t *source_bits, const uint32_t *target_bits,
                                  int32_t *nbr_out,
                                  uint32_t *tile_bits_out, int32_t *perm_out, int32_t *ctrl,
                                  void *ws, size_t ws_bytes, void *stream);

/* out[perm ? perm[r] : r] = epilogue(sum_p sources[nbr[p, r]] @ weights[order ? order[p] : p]) with
 * epilogue(v) = relu?(v * scale[c] + shift[c] + residual[t, c]); scale, shift
 * (fp32 [c_out]) and residual ([T, c_out], feature dtype) may each be NULL.
 * sub_tiles: 128-row sub-tiles per CTA tile (1..4; they share every weight tile);
 * 0 lets the library choose from pairs_per_row = (number of pairs) / T. */
size_t mn_implicit_workspace_bytes(int64_t O, int64_t c_in, int64_t c_out);
mn_status mn_sparse_convolution_forward_implicit(
    int64_t S, int64_t T, int64_t O, int64_t c_in, int64_t c_out, mn_dtype dtype,
    const void *sources, const void *weights, const void *weights_t, const int32_t *nbr,
    const uint32_t *tile_bits, const int32_t *perm, const int32_t *order, const float *scale, const float *shift,
    const void *residual, int relu, double pairs_per_row, int sub_tiles, void *targets_out,
    int32_t *status_dev, void *ws, size_t ws_bytes, void *stream);

/* weights_t_out[o, n, k] = weights[o, k, n]: the K-major weight layout the tensor-core
 * kernels read.  The three 16-bit forward entry points (implicit, pairs, dense) take
 * it as `weights_t`; with weights_t == NULL they transpose `weights` into their
 * workspace on every call, which is what a caller whose weights change between calls
 * wants.  No reference counterpart (the reference permutes its weights on every call,
 * sparse_convolution.cu:526-553). */
mn_status mn_transpose_weights(const void *weights, int64_t O, int64_t c_in, int64_t c_out,
                               mn_dtype dtype, void *weights_t_out, void *stream);

/* ---- Pair-list forward (sparse kernel maps) and dense forward ------------------ */
/* Same result as mn_sparse_convolution_forward followed by mn_apply_epilogue, for
 * fp16/bf16 and kernel maps that came out of mn_build_kernel_map with their hit
 * words (source_bits / target_bits).  It replaces the reference's gather,
 * bucket GEMMs, scatter and centre GEMM (sparse_convolution.cu:505-661) by:
 * a pair list built once per kernel map (mn_build_pair_list: the source row of
 * every product row; mask row p owns a 128-aligned block of mn_pair_rows rows in
 * total), one tensor-core kernel that multiplies the listed rows and keeps the
 * products in fp32, and the tensor-core GEMM of the centre offset (taken when
 * allow_shortcut != 0 and the last mask row is the identity) whose epilogue adds
 * each output row's other products, applies scale / shift / residual / ReLU and
 * rounds once.  No mask row is scanned; where a pair exists one mask word is
 * read.  Same shape limits as the fused implicit kernel. */
int mn_pairs_supported(int64_t O, int64_t c_in, int64_t c_out, mn_dtype dtype);
int64_t mn_pair_rows(const int32_t *sizes_host, int64_t O, int64_t S, int64_t T,
                     int allow_shortcut);
mn_status mn_build_pair_list(const int32_t *source_masks, const uint32_t *source_bits,
                             const int32_t *sizes_host, int64_t O, int64_t S, int64_t T,
                             int allow_shortcut, int32_t *pair_src_out, void *stream);
size_t mn_pairs_workspace_bytes(const int32_t *sizes_host, int64_t O, int64_t S, int64_t T,
                                int64_t c_in, int64_t c_out, int allow_shortcut);
mn_status mn_sparse_convolution_forward_pairs(
    int64_t S, int64_t T, int64_t O, int64_t c_in, int64_t c_out, mn_dtype dtype,
    const void *sources, const void *weights, const void *weights_t,
    const int32_t *target_masks, const uint32_t *target_bits, const int32_t *pair_src,
    const int32_t *order, const int32_t *sizes_host, int allow_shortcut, const float *scale,
    const float *shift, const void *residual, int relu, void *targets_out, int32_t *status_dev,
    void *ws, size_t ws_bytes, void *stream);

/* out = relu?((features @ weights) * scale + shift + residual) on the tensor cores:
 * the 1x1x1 convolution, for which the reference calls torch.mm
 * (minuet/nn/convolutions.py:448-454).  fp16/bf16, c_in a multiple of 8, c_out
 * even and at most 256; weights [c_in, c_out]; scale, shift, residual may be NULL. */
int mn_dense_supported(int64_t c_in, int64_t c_out, mn_dtype dtype);
size_t mn_dense_workspace_bytes(int64_t c_in, int64_t c_out);
mn_status mn_dense_forward(int64_t rows, int64_t c_in, int64_t c_out, mn_dtype dtype,
                           const void *features, const void *weights, const void *weights_t,
                           const float *scale, const float *shift, const void *residual, int relu,
                           void *out, int32_t *status_dev, void *ws, size_t ws_bytes,
                           void *stream);

/* The same product for every dtype and shape (fp32, channels that are not a multiple
 * of 8, c_out above 256) on the FFMA grouped-GEMM kernel, followed by the in-place
 * epilogue pass when one is asked for.  fp32 must not go through TF32 tensor cores:
 * their 10-bit mantissa breaks the 1e-5 bound.  Needs no workspace. */
mn_status mn_dense_forward_simt(int64_t rows, int64_t c_in, int64_t c_out, mn_dtype dtype,
                                const void *features, const void *weights, const float *scale,
                                const float *shift, const void *residual, int relu, void *out,
                                void *stream);

/* Per-voxel mean of point features for voxelisation (the reference's
 * minuet/nn/functional/voxelize.py:10-35 stops at the unique coordinates).
 * sorted_index [n]: the arg-sort of the floored points; run_ids [n] (the first n entries
 * of the unique op's index array): voxel of sorted row i, non-decreasing.
 * means_out[u, :] = mean over the points of voxel u, summed in fp32 in sorted order
 * (deterministic, no atomics).  features / means_out: [n, channels] / [U, channels]. */
mn_status mn_voxel_mean(const void *features, int64_t n, int64_t channels, mn_dtype dtype,
                        const int64_t *sorted_index, const int64_t *run_ids, void *means_out,
                        void *stream);

/* In place: features[t, c] = relu?(features[t, c] * scale[c] + shift[c] + residual[t, c]);
 * scale / shift (fp32 [channels]) and residual ([rows, channels], feature dtype)
 * may be NULL.  The same epilogue the fused forward applies inside its kernel,
 * for layers that go through gather - GEMM - scatter.  No reference counterpart
 * (the reference's models run BatchNorm, add and ReLU as separate torch ops). */
mn_status mn_apply_epilogue(void *features, int64_t rows, int64_t channels, mn_dtype dtype,
                            const float *scale, const float *shift, const void *residual,
                            int relu, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* MINUET_B200_H_ */
