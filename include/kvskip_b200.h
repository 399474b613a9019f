/*
 * kvskip_b200 -- C ABI of the sm_100a decode-attention library (libkvskip_b200.so).
 *
 * One entry point per launcher of the reference's kernel layer (kernels/kvskip.h:113-120 in
 * format37/kvskip), with the same parameter blocks: plain pointers, sizes and ELEMENT strides,
 * no framework types.  Differences from the reference's C++ launchers:
 *   - C linkage, the parameter block is passed by pointer, the stream as an opaque pointer
 *     (a cudaStream_t);
 *   - every call returns 0 on success or a negative KVSKIP_E_* code and never throws;
 *     kvskip_last_error() gives the message of the calling thread's last failure;
 *   - per-device set-up (shared-memory opt-in, scratch) is keyed by the current device, so one
 *     process can drive several GPUs.
 * Nothing is synchronised: kernels are enqueued on the given stream and the call returns.
 * All pointers are device pointers on the current device unless stated otherwise.
 */
#ifndef KVSKIP_B200_H_
#define KVSKIP_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KVSKIP_TILE 64 /* tokens per KV block: unit of the masks, of the statistics and of a load */

#define KVSKIP_OK 0
#define KVSKIP_E_ARG (-1)     /* unsupported shape / flag combination / misaligned pointer */
#define KVSKIP_E_CUDA (-2)    /* a CUDA runtime or driver call failed */
#define KVSKIP_E_LIMIT (-3)   /* size beyond a stated maximum */

/* Parameter block of the attention family.  Field meaning follows the reference's
 * kvskip::Params (kernels/kvskip.h:13-60); bf16 / fp16 tensors are typed as uint16_t. */
typedef struct kvskip_params {
  /* q [B,Hq,D]; k, v [B,Hkv,T,D], any batch / head / token strides, D contiguous, rows 16-byte
   * aligned */
  const uint16_t* q;
  const uint16_t* k;
  const uint16_t* v;
  int64_t q_sb, q_sh;
  int64_t k_sb, k_sh, k_st;
  int64_t v_sb, v_sh, v_st;
  int32_t B, Hq, Hkv, T;
  float scale_log2; /* softmax scale * log2(e) */

  /* masked mode: ascending list of blocks to read per (b, kv head); entries >= block_cnt ignored */
  const int32_t* block_idx; /* [B,Hkv,max_blocks] */
  const int32_t* block_cnt; /* [B,Hkv] */
  int32_t max_blocks;

  /* split-K: caller-provided scratch, needed when num_splits > 1 */
  int32_t num_splits;
  float* part_acc; /* [B,Hq,num_splits,D] un-normalised partial outputs, relative to the split max */
  float* part_ml;  /* [B,Hq,num_splits,2] split max (log2 units) and split sum */

  /* outputs */
  uint16_t* out;  /* bf16 [B,Hq,D] */
  float* out_f32; /* optional [B,Hq,D] */
  float* lse;     /* [B,Hq] natural-log log-sum-exp over the blocks read */

  /* block statistics: per query head and 64-token block */
  float* blk_max; /* [B,Hq,nb] max score, natural-log units, scale applied */
  float* blk_sum; /* [B,Hq,nb] sum exp(score - blk_max) */
  int32_t nb;

  /* two-pass V-skip */
  uint16_t* p_out;        /* fp16 [B,Hq,t_pad] exp(s - blk_max), written by a statistics pass, or NULL */
  const uint16_t* p_in;   /* fp16 [B,Hq,t_pad], read by the pv pass */
  const float* blk_scale; /* [B,Hkv,nb,G] exp(blk_max - lse_kept), 0 for dropped blocks */
  int64_t t_pad;          /* nb * KVSKIP_TILE */

  /* single-pass V-skip */
  float log2_tau;
  int32_t local;
  int32_t* vcount;       /* [B,Hkv] V blocks loaded, accumulated atomically; optional */
  const float* lse_prev; /* [B,Hq] natural-log normaliser estimate; NULL: bound by the sink block */
} kvskip_params;

/* Refresh planner, before the pass.  Follows kvskip::PlanParams (kernels/kvskip.h:63-89). */
typedef struct kvskip_plan_params {
  const uint16_t* q; /* bf16 [B,Hq,D] */
  int64_t q_sb, q_sh;
  const uint16_t* k; /* bf16 cache view [B,Hkv,T,D]; the token appended by this step sits at T-1 */
  int64_t k_sb, k_sh, k_st;
  float* csum;          /* [B,Hkv,NBC,D] per-block key sums, updated in place when add_token */
  const float* lse_ref; /* [B,Hq,NBC] block log-sum-exp at the head's last refresh (-inf: none) */
  const float* cs_ref;  /* [B,Hq,NBC] centroid scores at that refresh */
  const uint8_t* keep;  /* [B,Hkv,NBC] stored set */
  const float* lse_att; /* [B,Hq] previous step's log-sum-exp over the attended set */
  int32_t* age;         /* [B,Hkv] steps since the last refresh, updated */
  const int32_t* flags; /* [Hkv] bit 0 refresh every step, bit 1 token-index-only, bit 2 index union */
  const uint8_t* idx;   /* [B,NBC] this step's token-index blocks, or NULL */
  const float* calib;   /* [B,Hkv] correction of the estimate, or NULL */
  float* est;           /* [B,Hkv] out: uncorrected estimate (max over the group), or NULL */
  int32_t calib_on;
  int32_t calib_kind; /* 0 log-odds offset; 1, 2 added to the share */
  const uint8_t* aix; /* [B,Hkv] heads latched onto the token index, or NULL */
  float* cs_now;      /* [B,Hq,NBC] out: this step's centroid scores */
  uint8_t* trig;      /* [B,Hkv] out: refresh decision */
  int32_t* block_idx; /* [B,Hkv,NBC] out: blocks to read, ascending */
  int32_t* block_cnt; /* [B,Hkv] out */
  int32_t B, Hq, Hkv, T, NBC, local, max_age, add_token;
  float scale, delta;
} kvskip_plan_params;

/* Refresh planner, after the pass.  Follows kvskip::UpdateParams (kernels/kvskip.h:91-111). */
typedef struct kvskip_update_params {
  const float* blk_max; /* [B,Hq,nb] statistics of this step's pass (-inf / 0 on blocks not read) */
  const float* blk_sum;
  const uint8_t* trig;  /* [B,Hkv] */
  const float* cs_now;  /* [B,Hq,NBC] */
  uint8_t* keep;        /* [B,Hkv,NBC] updated for refreshing heads */
  float* lse_ref;       /* [B,Hq,NBC] updated for refreshing heads */
  float* cs_ref;        /* [B,Hq,NBC] updated for refreshing heads */
  float* lse_att;       /* [B,Hq] updated for every head */
  const int32_t* flags; /* [Hkv] */
  const uint8_t* idx;   /* [B,NBC] or NULL */
  const float* est;     /* [B,Hkv] */
  float* calib;         /* [B,Hkv] or NULL: no learning */
  float calib_rate;
  int32_t calib_free;
  int32_t calib_kind;
  uint8_t* aix; /* [B,Hkv] or NULL */
  float aix_thr;
  int32_t B, Hq, Hkv, T, NBC, local;
  float level;
} kvskip_update_params;

/* Split-K flash-decoding: dense, masked block list, block statistics, statistics only.
 * Replaces kvskip::launch_decode (kernels/kvskip.h:113; kernels/kvskip_kernel.cu:761-769).
 * Runs the split merge itself when num_splits > 1 and load_v.  `stages` is accepted for
 * compatibility (2 or 3); the ring depth is chosen by the library. */
int kvskip_launch_decode(const kvskip_params* p, int D, int G, int stages, int masked, int stats, int load_v,
                         void* stream);

/* The same launch for callers that cannot allocate device memory when they call: a serving
 * engine that hands out all of its memory at start-up and treats a later cudaMalloc as a bug, a
 * latency-critical loop that cannot afford the implicit synchronisation of an allocation, or a
 * plugin interface that only passes input and output buffers.  No counterpart in the reference,
 * whose binding allocates split scratch on every call.
 * Takes the same arguments as kvskip_launch_decode; p->part_acc and p->part_ml are ignored.
 * When num_splits > 1 the split partials go to an array built into the library (one per device
 * that loads it, held until exit) instead of caller scratch:
 *   - limit: B*Hq*num_splits*(D+2) <= KVSKIP_NOALLOC_MAX_FLOATS (1 Mi floats = 4 MiB), else
 *     KVSKIP_E_LIMIT with a message saying so;
 *   - the first call on a device looks the array's address up (cudaGetSymbolAddress, with that
 *     device current) and opts the kernel into its shared-memory size; make that first call
 *     during start-up, outside the latency-critical part of the host program;
 *   - all calls on a device share the array: two calls whose kernels overlap on the GPU (different
 *     streams) race on it; calls on one stream are ordered and safe.  The array keeps the last
 *     call's contents and nothing in it needs clearing.
 * Calls no cudaMalloc / cudaFree and no allocating library routine. */
#define KVSKIP_NOALLOC_MAX_FLOATS (1 << 20)
int kvskip_launch_decode_noalloc(const kvskip_params* p, int D, int G, int stages, int masked, int stats,
                                 int load_v, void* stream);

/* Single-pass V-skip.  Replaces kvskip::launch_vskip1 (kernels/kvskip.h:118;
 * kernels/kvskip_kernel.cu:747-752). */
int kvskip_launch_vskip1(const kvskip_params* p, int D, int G, void* stream);

/* Two-pass V-skip, second pass.  Replaces kvskip::launch_pv (kernels/kvskip.h:117;
 * kernels/kvskip_kernel.cu:754-759). */
int kvskip_launch_pv(const kvskip_params* p, int D, int G, void* stream);

/* Refresh planner.  Replace kvskip::launch_plan / launch_update (kernels/kvskip.h:115-116;
 * kernels/kvskip_planner.cu:309-318). */
int kvskip_launch_plan(const kvskip_plan_params* p, void* stream);
int kvskip_launch_update(const kvskip_update_params* p, void* stream);

/* Streaming read of `bytes` (multiple of 16) with `blocks` CTAs: the bandwidth-ceiling probe.
 * Replaces kvskip::launch_read (kernels/kvskip.h:120; kernels/kvskip_kernel.cu:738-740). */
int kvskip_launch_read(const void* x, int64_t bytes, uint32_t* out, int blocks, void* stream);

/* The same probe through the copy engine (no counterpart in the reference): every CTA streams
 * 32 KB pieces of x with bulk copies into a shared-memory ring, as the attention kernels load K/V
 * blocks, and discards them.  Reads floor(bytes / 32768) whole pieces; x 16-byte aligned.  One CTA
 * holds 192 KB of shared memory, so `blocks` = the number of SMs is the natural grid. */
int kvskip_launch_read_bulk(const void* x, int64_t bytes, uint32_t* out, int blocks, void* stream);

/* Dynamic shared memory of one decode CTA.  Replaces kvskip::max_smem_bytes
 * (kernels/kvskip.h:119; kernels/kvskip_kernel.cu:742-745). */
int kvskip_max_smem_bytes(int D, int stages, int load_v);

/* Merge of R partial results per row: the split merge of kernels/kvskip_kernel.cu:294-314 as an
 * entry point of its own, used for sequence shards gathered from several GPUs (the reference has
 * no multi-GPU path).  part_acc [R,N,D], part_ml [R,N,2] (max in log2 units, sum), merged in
 * ascending r; writes out (bf16, optional), out_f32 (optional), lse (optional) of N rows. */
int kvskip_launch_merge(const float* part_acc, const float* part_ml, int R, int64_t N, int D, uint16_t* out,
                        float* out_f32, float* lse, void* stream);

/* Sequence shards without intermediate tensor ops: pack a rank's normalised result (out_f32 [N,D],
 * lse [N]) into rows [acc(D) | m | l] = [out | lse/ln2 | 1] of `packed` [N,D+2] (the buffer handed
 * to the all-gather), and merge R gathered buffers `parts` [R,N,D+2] in ascending r. */
int kvskip_launch_pack_partial(const float* out_f32, const float* lse, float* packed, int64_t N, int D, void* stream);
int kvskip_launch_merge_packed(const float* parts, int R, int64_t N, int D, uint16_t* out, float* out_f32, float* lse,
                               void* stream);

/* Sequence shards, exchange and merge fused in one kernel over peer memory (no collective call).
 * Every rank (one process per GPU, R <= 8) passes its normalised local result (out_f32 [N,D],
 * lse [N]), the R peer-visible addresses of the ranks' exchange buffers, its rank, and a step
 * number seq that is the same on every rank and grows by one per call (starting at 1).
 * An exchange buffer holds 2*R*N*(D+2) words of 8 bytes (8-byte aligned, zero before the first
 * step): a word is (fp32 value, step number), written with one 8-byte store, so the flag travels
 * with the data and a reader polls the word itself -- no fence, no flag array, one NVLink crossing.
 * peer_flags is not used and may be null (kept for callers of the earlier flag-array protocol).
 * Each row is stored into every rank's buffer with plain stores over NVLink, awaited word by word
 * and merged in ascending rank order; results equal kvskip_launch_merge_packed on the all-gathered
 * buffers bit for bit.  The wait is bounded ("spin_limit" option, about two seconds by default); on
 * expiry the device status word is set and the missing rank counts as having read nothing.  All
 * ranks must call it for the same step: a rank that does not shows up as that timeout, not as a hang. */
int kvskip_launch_exchange_merge(const float* out_f32, const float* lse, float* const* peer_bufs,
                                 unsigned int* const* peer_flags, int rank, int R, int64_t N, int D, unsigned int seq,
                                 uint16_t* out, float* res_f32, float* res_lse, void* stream);

/* Sequence shards, everything in one kernel: kvskip_launch_decode whose split merge also does the
 * exchange of kvskip_launch_exchange_merge -- the CTA that merges the splits of a (batch, kv head)
 * stores the result as a packed triple into every rank's buffer (plain peer stores of (value, step)
 * words), waits (bounded, status word 0x510 + peer) for the peers' words and merges the R triples in
 * ascending rank order; p->out / out_f32 / lse receive the result over the whole sequence.  Same
 * buffers, seq convention and bits as kvskip_launch_exchange_merge (N = B * Hq rows).
 * Needs num_splits > 1, D = 128 and at most half as many (batch, kv head) pairs as SMs. */
int kvskip_launch_decode_xchg(const kvskip_params* p, int D, int G, int stages, int masked, int stats,
                              float* const* peer_bufs, unsigned int* const* peer_flags, int rank, int R,
                              unsigned int seq, void* stream);

/* Token-index blocks of one decode step on the device (the reference builds them with torch ops,
 * src/lab.py:149-167): ids int64 [n, ids_stride], current token at T-1; out uint8 [n, NBC], a
 * block is marked if it holds an earlier copy of the current token or the position after one. */
int kvskip_launch_index_blocks(const int64_t* ids, int64_t ids_stride, int n, int T, uint8_t* out, int NBC,
                               void* stream);

/* Device-resident sequence length (no counterpart in the reference, whose launches take T by value;
 * its README lists a captured decode step as an open item).  The same kernels as the entry points
 * above, but the length they work on is read from *t_dev on the device after the preceding work
 * of the stream has finished, so one captured sequence of launches can be replayed while the
 * cache grows.  The T of the parameter block (T_bound for the index) is then an upper bound: it
 * sizes the grid, the tensor maps (the K/V views must be valid for T rows) and the layout -- the
 * statistics rows keep the stride ceil(T/64), and blocks between the current and the bounded
 * length are reported as unread (-inf / 0).  A value outside [1, T] is clamped.  K/V rows beyond
 * the current length are never used, whatever they hold.  Tensor-core path only (D = 128).
 * kvskip_launch_advance adds delta to *t_dev in stream order (one thread). */
int kvskip_launch_decode_dyn(const kvskip_params* p, int D, int G, int stages, int masked, int stats, int load_v,
                             const int* t_dev, void* stream);
int kvskip_launch_plan_dyn(const kvskip_plan_params* p, const int* t_dev, void* stream);
int kvskip_launch_update_dyn(const kvskip_update_params* p, const int* t_dev, void* stream);
int kvskip_launch_index_blocks_dyn(const int64_t* ids, int64_t ids_stride, int n, int T_bound, const int* t_dev,
                                   uint8_t* out, int NBC, void* stream);
int kvskip_launch_advance(int* t_dev, int delta, void* stream);
/* The V-skip entry points with the length on the device (tensor-core path, D = 128): the single
 * pass, the second pass of the two-pass form, and the selection between its passes (T_bound sizes
 * the rows of blk_max / blk_sum / keep / block_idx / weight: ceil(T_bound / 64) blocks; entries of
 * keep and weight beyond the current length are written as zero). */
int kvskip_launch_vskip1_dyn(const kvskip_params* p, int D, int G, const int* t_dev, void* stream);
int kvskip_launch_pv_dyn(const kvskip_params* p, int D, int G, const int* t_dev, void* stream);
int kvskip_launch_select_dyn(const float* blk_max, const float* blk_sum, int B, int Hkv, int T_bound, const int* t_dev,
                             int rule, float value, int local, uint8_t* keep, int32_t* block_idx, int32_t* block_cnt,
                             float* weight, void* stream);

/* Block selection between the two passes of the two-pass V-skip, in one launch (the reference's
 * caller does it with torch ops: kernels/kvskip.py:122-147 select_blocks, :165-177, :70-85
 * make_plan).  blk_max, blk_sum fp32 [B,4*Hkv,nb] from the statistics pass; rule 0: per query head
 * the heaviest blocks whose softmax mass reaches `value` (top-p), rule 1: blocks of weight >=
 * `value`; a kv head keeps the union over its four heads plus block 0 and the `local` newest.
 * Outputs: keep u8 [B,Hkv,nb], block_idx int32 [B,Hkv,nb] (ascending) with block_cnt [B,Hkv], and
 * weight fp32 [B,Hkv,nb,4] = exp(blk_max - log-sum-exp of the kept blocks), 0 where not kept: the
 * blk_scale of kvskip_launch_pv. */
int kvskip_launch_select(const float* blk_max, const float* blk_sum, int B, int Hkv, int nb, int rule, float value,
                         int local, uint8_t* keep, int32_t* block_idx, int32_t* block_cnt, float* weight,
                         void* stream);

/* Paged cache (no counterpart in the reference, which reads [B,Hkv,T,D] views; its notes name a
 * cache in which a 64-token block is a page as the natural layout next to the block lists).
 * k and v of the parameter block are page pools [num_pages, Hkv, 64, D] (k_sb = page stride, k_sh,
 * k_st as usual, D contiguous); page_table int32 [B, max_pages] names the page of every 64-token
 * block of every sequence, max_pages >= ceil(T/64).  Block lists, statistics and planner state keep
 * their per-sequence block numbering.  An entry outside the pool reads as zeros in the attention
 * kernel and is skipped (status word 0x300 / 0x301) where a single row is addressed.  t_dev may be
 * null (length by value) or a device-resident length as above.  Tensor-core path only (D = 128);
 * write_p is not supported.  `update` and the token index do not touch K/V and need no variant.
 * kvskip_launch_vskip1_paged is the single-pass V-skip over the same pools (length by value).
 * kvskip_launch_append writes the K and V rows of the newest token (row T-1, T the length after
 * the append) from k_new, v_new [B,Hkv,D] into a contiguous cache (page_table null; sb, sh, st its
 * element strides) or into the pool. */
int kvskip_launch_decode_paged(const kvskip_params* p, int D, int G, int stages, int masked, int stats, int load_v,
                               const int32_t* page_table, int max_pages, int num_pages, const int* t_dev,
                               void* stream);
int kvskip_launch_plan_paged(const kvskip_plan_params* p, const int32_t* page_table, int max_pages, int num_pages,
                             const int* t_dev, void* stream);
int kvskip_launch_vskip1_paged(const kvskip_params* p, int D, int G, const int32_t* page_table, int max_pages,
                               int num_pages, void* stream);
int kvskip_launch_append(uint16_t* k, uint16_t* v, int64_t sb, int64_t sh, int64_t st, const uint16_t* k_new,
                         const uint16_t* v_new, int B, int Hkv, int D, int T, const int* t_dev,
                         const int32_t* page_table, int max_pages, int num_pages, void* stream);

/* Process-wide options (no counterpart in the reference).
 *   "decode_path"  0 (default): tensor-core kernel for D = 128, exact-order kernel otherwise;
 *                  1: exact-order kernel everywhere -- scores, block statistics and outputs are
 *                     bit-identical to the reference's kernels on the same GPU;
 *                  2: tensor-core kernel, error where it does not exist.
 *   "half_cta"     1 (default): when a dense (no block list) tensor-core decode launch has at least
 *                  four CTAs per SM of the GPU it uses CTAs of half the size (3 consumer warps, 3 stages), two per SM, so the
 *                  set-up and merge of one overlap the streaming of the other; 0: always one
 *                  full-size CTA per SM.
 *   "pdl"          1 (default): the attention and planner kernels are launched with programmatic
 *                  stream serialisation, so their set-up overlaps the tail of the previous kernel
 *                  on the stream (they wait for it before reading memory); 0: plain launches.
 *   "queue"        1 (default): a decode launch with block lists, V loaded, 32 to 1024 (batch, kv head)
 *                  pairs and more pieces than SMs runs as one persistent CTA per SM pulling (head,
 *                  piece) items from a device-side queue; 0: one CTA per piece.  Same bits either way.
 *   "queue_min_heads"  fewest (batch, kv head) pairs of a launch that takes the queue kernel; default 32.
 *   "min_blocks"   shortest piece (in 64-token blocks) a block list is cut into when the launch has
 *                  more CTAs than SMs; default 24.
 *   "plan_cluster" CTAs per (batch, kv head) of `plan` when it runs on thread-block clusters (the CTAs
 *                  of a head hand their results to the first one through its shared memory): 1, 2, 4 or
 *                  8; -1 (default): chosen per launch, about four CTAs per SM; 0: the version that
 *                  counts a head's finished CTAs in global memory (also used, whatever the option,
 *                  beyond 12 000 blocks, where a head's table no longer fits in shared memory).
 *   "plan_rounds"  32-block rounds per CTA of that counter version: 1, 2, 4 or 8; 0 (default): chosen
 *                  per launch.  Every setting of these two leaves every output of `plan` bit-identical.
 *   "spin_limit"   polls (about 100 ns each) a kernel of the sequence-sharded exchange spends on a
 *                  peer's flag before it gives up, sets the status word (0x500 + peer from
 *                  kvskip_launch_exchange_merge, 0x510 + peer from kvskip_launch_decode_xchg),
 *                  merges what arrived and returns; default 2^21 (about 2 s); 0 restores it.
 *
 * Concurrency.  The kernels that merge their splits in the same launch (attention, V-skip, the
 * counter version of plan) count finished CTAs in device counters owned by the (device, stream) pair of the launch: launches
 * on one stream follow one another and share them safely, launches on different streams use
 * different ones, and a launch captured into a CUDA graph keeps the counters of the stream it was
 * captured on.  Unsupported: replaying such a graph while other launches of this library run on the
 * stream it was captured on.  A device that has used more than 64 streams with this library gets a
 * separate merge launch for the newcomers (plan reports KVSKIP_E_LIMIT). */
int kvskip_set_option(const char* name, int value);
int kvskip_get_option(const char* name);

/* Message of the calling thread's last failed call ("" if none). */
const char* kvskip_last_error(void);

/* Reads (and clears) the current device's kernel status word after synchronising `stream`:
 * 0 if every bounded wait inside the kernels completed, otherwise the code of the first that
 * gave up (0x2xx / 0x4xx: a stage of a kernel's load ring; 0x300 / 0x301: a page table entry outside
 * the pool; 0x310: plan's hand-over inside a cluster; 0x500 + peer, 0x510 + peer: the exchange between
 * GPUs).  Host-blocking; meant for tests and post-mortems, not for the hot path.  When the word is
 * non-zero the call also waits for the whole device and clears the split counters a kernel that
 * gave up may have left behind: no launch of this library may be in flight on another host thread. */
int kvskip_device_status(void* stream, unsigned int* status);

/* Library version: major * 10000 + minor * 100 + patch. */
int kvskip_version(void);

#ifdef __cplusplus
}
#endif
#endif /* KVSKIP_B200_H_ */
