// homcomp-b200: public C API.
//
// Layers
//   hc_cpu_*      portable codec / homomorphic add / host-rank ring (the oracle)
//   hc_*          sm_100a device codec working on a caller-owned workspace (no allocation, no host
//                 sync; sizes are produced in device memory)
//   hc_comm_* / hc_allreduce_*   compressed collectives over peer-mapped buffers
// The names and signatures of the reference library (GSZ_*, homomorphic_sum*, allreduce_ring_*,
// cpuCopy_*, mixed_compressed_allreduce) are declared in homcomp_compat.h on top of these.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- format helpers ------------------------------------------------------------------------
size_t hc_max_compressed_bytes(size_t n);  // capacity that cannot overflow (129 B per block)
size_t hc_rate_bytes(size_t n);            // length of section A

// mode: 0 outlier codec, 1 plain codec, 2 stride-4 "vec" variant.  All functions return 0 on
// success or a hc::Status code.

// ---- CPU oracle ----------------------------------------------------------------------------
int hc_cpu_quantize(const float* x, size_t n, float eb, int32_t* q);
int hc_cpu_dequantize(const int32_t* q, size_t n, float eb, float* x);
int hc_cpu_quant_pred(const float* x, size_t n, float eb, int mode, int32_t* deltas);
int hc_cpu_compress(const float* x, size_t n, float eb, int mode, uint8_t* out, size_t cap, size_t* size);
int hc_cpu_decompress(const uint8_t* in, size_t size, size_t n, float eb, int mode, float* x);
int hc_cpu_decode_quant(const uint8_t* in, size_t size, size_t n, int mode, int32_t* q);
int hc_cpu_hom_add_f32(const uint8_t* in, size_t in_size, const float* local, size_t n, float eb, int mode,
                       uint8_t* out, size_t cap, size_t* size);
int hc_cpu_hom_add_i32(const uint8_t* in, size_t in_size, const int32_t* deltas, size_t n, int mode, uint8_t* out,
                       size_t cap, size_t* size);
int hc_cpu_hom_add_stream(const uint8_t* a, size_t a_size, const uint8_t* b, size_t b_size, size_t n, int mode,
                          uint8_t* out, size_t cap, size_t* size);
int hc_cpu_stream_size(const uint8_t* in, size_t avail, size_t n, size_t* size);

// Ring allreduce of P host buffers simulated in one process (rank r owns bufs[r], `count` floats
// each).  Results are written to outs[r].  hop_bytes (optional, P*P entries) receives the size of
// the stream rank r produced at step s as hop_bytes[r*P + s]; step P-1 is the reduced chunk that
// the all-gather distributes.  Partition and hop order are those of the device ring.
int hc_cpu_ring_allreduce(const float* const* bufs, float* const* outs, int P, size_t count, float eb,
                          size_t* hop_bytes);
// Chunk geometry of the collectives: `count` floats over P ranks, chunk length rounded up to
// whole 32-element blocks.  Returns the chunk length in elements.
size_t hc_chunk_elems(size_t count, int P);

// ---- sm_100a device codec -----------------------------------------------------------------------
// All pointers below are device pointers unless named otherwise.  Calls only enqueue work on
// `stream`: they never allocate, never synchronise and never copy to the host.  The exact stream
// length is written to the device word d_size.  One codec handle serialises on one stream at a
// time (its workspace holds the look-back state of the launch in flight).
// Input streams are read with 16-byte aligned bulk copies: the buffer that holds a stream must be
// readable up to the next 16-byte boundary past its last byte (true of any device allocation whose
// size is a multiple of 16, e.g. one of hc_max_compressed_bytes(n) rounded up).
typedef struct CUstream_st* hc_stream_t;  // same type as cudaStream_t
typedef struct hc_codec hc_codec;

size_t hc_codec_workspace_bytes(size_t max_elems);
// Workspace owned by the handle (one cudaMalloc here, at set-up time).
int hc_codec_create(hc_codec** out, size_t max_elems);
// Workspace provided by the caller (d_workspace of at least hc_codec_workspace_bytes(max_elems));
// it is zeroed once on `stream`.
int hc_codec_create_in(hc_codec** out, void* d_workspace, size_t bytes, size_t max_elems, hc_stream_t stream);
void hc_codec_destroy(hc_codec* c);
// Upper bound for every device-side wait (look-back, arrival flags, TMA barriers); default 2000 ms.
int hc_codec_set_timeout_ms(hc_codec* c, unsigned ms);
// Synchronises the device, returns the sticky hc::Status of the handle and clears it when asked.
int hc_codec_status(hc_codec* c, int clear);
// After a status 3 (time-out): which wait ran out FIRST in the launch that failed (call it before
// clearing the status).  1 loader: fp32 stage not released, 2 loader: input buffer not released,
// 3 compute: input stream not staged, 4 compute: fp32 tile not landed, 5 compute: no room in the
// payload ring, 6 scanner: tile total missing, 7 copier: look-back result missing, 8 copier: tile not
// packed, 9 / 10 the decoder's loader / compute warps, 11 a look-back over tile totals; 0 none.
int hc_codec_status_site(hc_codec* c);
// Stand-alone decompress / homomorphic adds on large streams (16 MiB of values and up) first run a
// small kernel that turns the input's rate bytes into per-tile payload offsets, so the main kernel
// stages every tile without a look-back over the input (two launches instead of one; on by
// default).  0 turns it off: one launch, input offsets by decoupled look-back.  Same output bytes.
int hc_codec_set_prepass(hc_codec* c, int on);

int hc_compress(hc_codec* c, const float* d_x, size_t n, float eb, int mode, uint8_t* d_out, size_t cap,
                uint64_t* d_size, hc_stream_t stream);
int hc_decompress(hc_codec* c, const uint8_t* d_in, size_t in_size, size_t n, float eb, int mode, float* d_x,
                  hc_stream_t stream);
// Streaming decode: the stream is being written by another producer (another stream, another GPU).
// d_tile_flags holds one uint64 per tile of hc_tile_elems() values; tile t is decoded once the
// producer has stored (with release semantics at system scope)
//     d_tile_flags[t] = ((uint64_t)want << 40) | byte offset of the tile's payload in the stream
// where want is a non-zero 24-bit tag of the producer's choice (an offset field of all ones marks a
// tile the producer gave up on).  A flag that never rises ends in status 6 (peer) after the
// handle's timeout; the kernel always runs to its end.
int hc_decompress_flagged(hc_codec* c, const uint8_t* d_in, size_t in_size, size_t n, float eb, int mode, float* d_x,
                          const uint64_t* d_tile_flags, uint32_t want, hc_stream_t stream);
size_t hc_tile_elems(void);
// n_in (1..8) streams of the same n values, decoded and added in the quantised domain by one kernel:
// d_x = (q_1 + ... + q_n_in) * 2 eb, the values a chain of homomorphic adds followed by hc_decompress
// would give, without the intermediate streams.  Outlier / plain streams.
int hc_decompress_sum(hc_codec* c, int n_in, const uint8_t* const* d_in, const size_t* in_size, size_t n, float eb,
                      float* d_x, hc_stream_t stream);
int hc_hom_add_f32(hc_codec* c, const uint8_t* d_in, size_t in_size, const float* d_local, size_t n, float eb,
                   int mode, uint8_t* d_out, size_t cap, uint64_t* d_size, hc_stream_t stream);
// d_deltas: hc_quant_pred output, padded to whole 32-element blocks
int hc_hom_add_i32(hc_codec* c, const uint8_t* d_in, size_t in_size, const int32_t* d_deltas, size_t n, int mode,
                   uint8_t* d_out, size_t cap, uint64_t* d_size, hc_stream_t stream);
int hc_hom_add_stream(hc_codec* c, const uint8_t* d_a, size_t a_size, const uint8_t* d_b, size_t b_size, size_t n,
                      int mode, uint8_t* d_out, size_t cap, uint64_t* d_size, hc_stream_t stream);
// Up to 8 independent tensors compressed by one launch; out[g] needs cap_each bytes, d_sizes[g]
// receives the stream length.  The tensors together (each rounded up to whole 32768-value chunks)
// must fit the handle's max_elems.
int hc_compress_batch(hc_codec* c, int n_seg, const float* const* d_x, const size_t* n, float eb, int mode,
                      uint8_t* const* d_out, size_t cap_each, uint64_t* d_sizes, hc_stream_t stream);
// Sum of up to 8 streams and one fp32 operand in the quantised domain, encoded once.  n_in * n must
// fit the handle's max_elems.
int hc_hom_add_multi(hc_codec* c, int n_in, const uint8_t* const* d_in, const size_t* in_size, const float* d_local,
                     size_t n, float eb, int mode, uint8_t* d_out, size_t cap, uint64_t* d_size, hc_stream_t stream);
int hc_quant_pred(const float* d_x, size_t n, float eb, int mode, int32_t* d_deltas, hc_stream_t stream);
// dst = a + b (+ c) (+ d); c and d may be null; dst may alias a
int hc_sum(float* d_dst, const float* d_a, const float* d_b, const float* d_c, const float* d_d, size_t n,
           hc_stream_t stream);
const char* hc_status_string(int status);

// ---- compressed collectives over peer-mapped memory ------------------------------------------
// One process (or thread) per GPU.  Every rank provides a zeroed "symmetric" device region of
// hc_comm_symmetric_bytes() bytes that all other ranks can address (CUDA IPC mapping, a symmetric
// heap, peer access inside one process); peer_bases[r] is rank r's region as seen from this rank.
// All data movement is done by the kernels themselves with peer stores; there is no MPI or NCCL
// call on this path.  Counterpart of allreduce_ring_comprs_hom_sum_F
// (HomComp/src/cuda_awareallreduce.cu:166-264).
typedef struct hc_comm hc_comm;
size_t hc_comm_symmetric_bytes(int world, size_t max_count);
// mc_base: multicast (NVLS) mapping of the same region, or NULL to use peer stores only
int hc_comm_create(hc_comm** out, int rank, int world, size_t max_count, void* const* peer_bases, void* mc_base);
void hc_comm_destroy(hc_comm* c);
int hc_comm_set_timeout_ms(hc_comm* c, unsigned ms);
int hc_comm_status(hc_comm* c, int clear);  // synchronises; sticky hc::Status of all the handle's kernels
int hc_comm_status_site(hc_comm* c);        // after a time-out: the wait that ran out first (see hc_codec_status_site)
// Sum of `count` floats over all ranks, error at most world * eb per value; d_sbuf and d_rbuf may
// alias.  Enqueues 3 kernels (direct algorithm, the default; 2 for the small messages that take its
// one-step form, see hc_comm_set_small_count) or world + 1 (ring) on `stream`; never allocates or
// synchronises.
int hc_allreduce(hc_comm* c, const float* d_sbuf, float* d_rbuf, size_t count, float eb, hc_stream_t stream);
// The same sum for buffers in (pinned) host memory: the message crosses PCIe in `pieces` pieces
// (0 = default: pieces of 4 MiB, at most 16; never more than 32) on two copy streams of the handle while earlier pieces are reduced on
// `stream` and still earlier ones travel back, so the call costs about one direction of the
// transfer.  `stream` ends behind the last copy down.  The first call allocates the device staging
// (2 x max_count floats).  Pageable host memory works but serialises the copies.
int hc_allreduce_host(hc_comm* c, const float* h_sbuf, float* h_rbuf, size_t count, float eb, int pieces,
                      hc_stream_t stream);
// algorithm 0: ring reduce-scatter with one fused kernel per hop (world + 1 launches);
// algorithm 1 (default): direct scatter -> reduce -> gather for a switched fabric (3 launches).
// Both produce byte-identical reduced streams, hence bit-identical results.
// algorithm 2: one step (2 launches) for every message of at most max_count / world values (larger ones
// take the direct form): every rank broadcasts its whole compressed message and decodes the sum of
// all streams.  Same result bits again; world - 1 messages on the wire instead of 2 (world - 1) / world.
int hc_comm_set_algorithm(hc_comm* c, int algorithm);
// Direct algorithm: messages of at most `count` values that fit one stream slot (max_count / world
// values; max_count with two ranks) take the one-step form, which has one network phase less.
// Default: 12 Mi values with 2 ranks, 1.5 Mi with 3 or 4, 512 Ki above; 0: never.
int hc_comm_set_small_count(hc_comm* c, size_t count);
// The form the last hc_allreduce took: 0 ring, 1 direct, 2 one step.  hc_comm_last_stream_bytes reports
// one stream per step of that form (one step: the whole message's stream in word 0, zeros behind it).
int hc_comm_last_form(hc_comm* c);
// Direct algorithm: launch steps 2 and 3 with programmatic stream serialisation, so that each fills
// the SMs while its predecessor drains (default on; off while tracing).  Same results either way.
int hc_comm_set_overlap(hc_comm* c, int on);
// Direct algorithm with overlap on: how many CTAs per SM step 1 (scatter-compress) and step 2
// (reduce) may take, so that the three steps of a call run side by side on the GPU, each consuming
// the tiles of the one before as their flags arrive, instead of one after the other (0: no limit,
// every step takes the whole GPU as it becomes free).  reduce_variant: 0 launcher's choice, 1 the
// add kernel with the payload ring, 2 the in-place one.  Results do not depend on any of it.
int hc_comm_set_shares(hc_comm* c, int scatter_ctas_per_sm, int reduce_ctas_per_sm, int reduce_variant);
// Transport buffers between the steps of a call: tiles at fixed offsets, as if every block before
// them were incompressible (default), or packed back to back as in a stored stream (0).  With fixed
// offsets no CTA waits for a prefix over other CTAs' tiles; the buffers are sized for the worst case
// either way, only the bytes of the payload are ever written or read, and consumers take each tile's
// offset from its arrival flag.  Results and hc_comm_last_stream_bytes do not depend on it.
int hc_comm_set_sparse_tiles(hc_comm* c, int on);
// Uncompressed sum over the same peer mappings (two-shot direct algorithm, three kernels); the
// compressed and the uncompressed collective of one handle must not be in flight together.
int hc_allreduce_raw(hc_comm* c, const float* d_sbuf, float* d_rbuf, size_t count, hc_stream_t stream);
// Hierarchical allreduce for ranks that form groups (nodes, or halves of one NVSwitch box): raw fp32
// reduce-scatter inside the group of `local`, hc_allreduce (error bound eb) of this rank's slice of
// the group sum over `inter` (the ranks with the same local index in the other groups; NULL or a
// world of 1: one group, nothing is compressed), raw all-gather inside the group.  The result is
// identical on every rank of every group.  inter must take hc_chunk_elems(count, local world) values.
// Seven kernels on `stream` (4 raw + the 3 of hc_allreduce); the first call allocates the slice buffer.
int hc_allreduce_mixed(hc_comm* local, hc_comm* inter, const float* d_sbuf, float* d_rbuf, size_t count, float eb,
                       hc_stream_t stream);
// Attaches `inter` to `local` for the reference-named mixed_compressed_allreduce (homcomp_compat.h),
// whose signature has room for one communicator only.
int hc_comm_set_inter(hc_comm* local, hc_comm* inter);
hc_comm* hc_comm_get_inter(hc_comm* local);
// Recovery after a call that not every rank made (a rank raised an error on the host, skipped a
// step, was restarted): the others' kernels run into their time-out and report status 6, nothing
// hangs.  To go on, every rank reads its call numbers, the ranks agree on the element-wise maximum
// over their host channel, every rank sets it with hc_comm_resync (synchronises the device) and
// clears its status; the next hc_allreduce is then an ordinary one.
int hc_comm_call_numbers(hc_comm* c, uint32_t out[2]);  // [0] compressed calls, [1] uncompressed / hierarchical calls
int hc_comm_resync(hc_comm* c, uint32_t call, uint32_t raw_call);
// Tracing: with trace on, hc_allreduce records one CUDA event per step; hc_comm_last_step_ms returns
// the device time of each step of the last call (reduce-scatter steps, then the decode).
int hc_comm_set_trace(hc_comm* c, int on);
int hc_comm_last_step_ms(hc_comm* c, float* ms, int n);
// device-side counters of the last call: bytes[s] = stream bytes this rank produced at step s
int hc_comm_last_stream_bytes(hc_comm* c, uint64_t* bytes, int n);

// ---- host-staged compressed allreduce (GPUs that cannot address each other) ---------------------
// The codec and the fused add run on the device; every compressed chunk goes through pinned host
// memory and the caller's transport.  send/recv move one message to / from rank dst / src and
// return 0 on success (recv stores the message length in *bytes; a message never exceeds cap).
// Ranks with an even number send first, the others receive first, so a blocking transport is
// fine.  Synchronises the host once per hop, like the reference's cpuCopy_* variants
// (HomComp/src/nca_allreduce.cu:195-324); its bounce buffers are allocated on the codec handle's first
// call and kept (the reference allocates them per call).  `codec` must have been
// created for at least hc_chunk_elems(count, world) values.
typedef int (*hc_send_fn)(void* user, int dst, const void* buf, size_t bytes);
typedef int (*hc_recv_fn)(void* user, int src, void* buf, size_t cap, size_t* bytes);
typedef struct hc_host_transport {
  hc_send_fn send;
  hc_recv_fn recv;
  void* user;
} hc_host_transport;
int hc_allreduce_host_staged(hc_codec* codec, const hc_host_transport* t, int rank, int world, const float* d_sbuf,
                             float* d_rbuf, size_t count, float eb, hc_stream_t stream);
// Registers the transport that the cpuCopy_* names of homcomp_compat.h use with this communicator.
int hc_comm_set_host_transport(hc_comm* c, const hc_host_transport* t);
int hc_comm_allreduce_host_staged(hc_comm* c, const float* d_sbuf, float* d_rbuf, size_t count, float eb,
                                  hc_stream_t stream);

// Symmetric regions with an NVSwitch multicast alias, built with the driver's virtual memory API
// (cuMemCreate / cuMulticastCreate / AddDevice / BindMem): what hc_comm_create takes as peer_bases
// and mc_base when the reduced chunks should leave with one multimem.st for all ranks and the
// uncompressed sum should be formed inside the switch.  hc_mc_create_local: one process drives all
// GPUs.  hc_mc_create_shared: one process per GPU (its current device); collective over `world`
// ranks that pass the same `session` string, handles travel as file descriptors over a unix-domain
// socket with rank 0 as the hub.  Regions come back zeroed.  Where a GPU lacks multicast support the
// regions are still mapped on every GPU and hc_mc_multicast_ptr returns NULL (peer stores then).
// All ranks must call hc_mc_destroy together, after a barrier of their own.
typedef struct hc_mc_region hc_mc_region;
int hc_multicast_supported(int device);
int hc_mc_create_local(hc_mc_region** out, int n_dev, const int* devices, size_t bytes);
int hc_mc_create_shared(hc_mc_region** out, int rank, int world, size_t bytes, const char* session);
void* hc_mc_unicast_ptr(hc_mc_region* r, int idx);  // region of GPU / rank idx as addressable from here
void* hc_mc_multicast_ptr(hc_mc_region* r);         // multimem instructions only; NULL without multicast
size_t hc_mc_bytes(hc_mc_region* r);
void hc_mc_destroy(hc_mc_region* r);
// CUDA IPC helpers for the multi-process bootstrap (the 64-byte handle travels over any host
// channel: torch.distributed, MPI, a file)
int hc_ipc_alloc(void** d_ptr, size_t bytes, uint8_t handle[64]);
int hc_ipc_open(const uint8_t handle[64], void** d_ptr);
int hc_ipc_close(void* d_ptr);
int hc_ipc_free(void* d_ptr);

#ifdef __cplusplus
}
#endif
