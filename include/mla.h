// Multi-head Latent Attention host API.
//
// The first four functions are drop-ins for the reference's include/mla.h
// (forward :18, backward :35, workspace size :57, paged decode :65): same names,
// argument order, layouts and error behaviour.  The prefill functions below
// them have no counterpart in the reference; they cover the non-absorbed form
// (per-head k_nope / v, one shared k_pe head) in dense and packed layouts.
//
// Every function only launches work on `stream`: no allocation, no
// synchronisation, no host read-back, so a call can be captured in a CUDA
// graph.  Bad arguments throw std::invalid_argument, CUDA failures throw
// std::runtime_error (as the reference's CUDA_CHECK does).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstddef>

namespace dscuda {

constexpr int MLA_KV_RANK = 512;
constexpr int MLA_ROPE_SIZE = 64;
constexpr int MLA_NOPE_SIZE = 128;
constexpr int MLA_VALUE_SIZE = 128;
// Bytes of one token row in the FP8 cache: 512 e4m3 values, four fp32 scales (one per 128
// columns), 64 bf16 rotary values.
constexpr int MLA_FP8_CACHE_ROW_BYTES = 512 + 16 + 128;

// Absorbed-query causal forward.  query_latent [B,T,H,C], query_rope [B,T,H,R],
// kv_latent [B,T,C] and key_rope [B,T,R] shared by all heads, output [B,T,H,C],
// logsumexp [B,H,T] (natural log, scale included).  C=512, R=64 only; B, T, H
// are free.
void mla_compressed_attention_forward_cuda(
    __nv_bfloat16* output,
    float* logsumexp,
    const __nv_bfloat16* query_latent,
    const __nv_bfloat16* query_rope,
    const __nv_bfloat16* kv_latent,
    const __nv_bfloat16* key_rope,
    int batch_size,
    int sequence_length,
    int heads,
    int kv_rank,
    int rope_size,
    float scale,
    cudaStream_t stream = nullptr);

// Backward of the above from the saved FP32 logsumexp.  The four gradient
// buffers (BF16, shapes of the matching inputs) are overwritten.
void mla_compressed_attention_backward_cuda(
    __nv_bfloat16* query_latent_gradient,
    __nv_bfloat16* query_rope_gradient,
    __nv_bfloat16* kv_latent_gradient,
    __nv_bfloat16* key_rope_gradient,
    const __nv_bfloat16* output_gradient,
    const __nv_bfloat16* output,
    const float* logsumexp,
    const __nv_bfloat16* query_latent,
    const __nv_bfloat16* query_rope,
    const __nv_bfloat16* kv_latent,
    const __nv_bfloat16* key_rope,
    int batch_size,
    int sequence_length,
    int heads,
    int kv_rank,
    int rope_size,
    float scale,
    cudaStream_t stream = nullptr);

// FP32 elements the caller must provide as decode workspace:
// B * H * splits * (C + 2).
std::size_t mla_decode_workspace_elements(
    int batch_size,
    int heads,
    int splits,
    int kv_rank);

// One packed BF16 query token [B,1,H,C+R] per sequence against a paged cache
// [blocks,page,1,C+R]; block_table [B,pages_per_sequence] holds physical page
// ids, cache_lengths [B] the number of valid tokens.  output [B,1,H,C],
// logsumexp [B*H].  page_size must be a multiple of 64.  `splits` bounds how
// many partial results per (sequence, head) the workspace can hold.
// A length of 0 gives NaN output and -inf logsumexp for that sequence (the
// softmax of an empty row); a length above pages_per_sequence * page_size is
// read as that capacity.  Page numbers are trusted: this signature (the
// reference's) does not carry the size of the cache.
void mla_decode_forward_cuda(
    __nv_bfloat16* output,
    float* logsumexp,
    const __nv_bfloat16* query,
    const __nv_bfloat16* paged_kv_cache,
    const int* block_table,
    const int* cache_lengths,
    float* workspace,
    int batch_size,
    int heads,
    int kv_rank,
    int rope_size,
    int page_size,
    int pages_per_sequence,
    int splits,
    float scale,
    cudaStream_t stream = nullptr);

// No counterpart in the reference.  mla_decode_forward_cuda for callers that know
// how many physical pages the cache has (`cache_blocks`): a block-table entry
// outside [0, cache_blocks) is read as page 0 and sets the device status to 3
// instead of reaching memory outside the cache.
void mla_decode_forward_checked_cuda(
    __nv_bfloat16* output,
    float* logsumexp,
    const __nv_bfloat16* query,
    const __nv_bfloat16* paged_kv_cache,
    const int* block_table,
    const int* cache_lengths,
    float* workspace,
    int batch_size,
    int heads,
    int kv_rank,
    int rope_size,
    int page_size,
    int pages_per_sequence,
    int cache_blocks,
    int splits,
    float scale,
    cudaStream_t stream = nullptr);

// Paged decode for callers that cannot hand over a workspace (no counterpart in
// the reference).  Same arguments and results as mla_decode_forward_cuda minus
// `workspace`: the split partials go to a fixed array inside the library image
// instead.  It is meant for hosts that may not allocate device memory at the
// point of the call - a serving loop whose memory pool is sized up front and
// handed out in full, a plugin that runs inside someone else's allocator, code
// that runs where cudaMalloc would stall every stream on the device.  Nothing
// is allocated or freed here, by CUDA or by any library.
//
// Limits and rules:
//   * batch_size * heads * splits must not exceed mla_decode_static_capacity()
//     (8192 partials, 16.1 MiB held by every GPU that loads the library, until
//     the process exits); larger requests throw std::invalid_argument.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress with that device current).  Make that first call
//     outside any stream capture.
//   * Every call on a device uses the same array.  Nothing in it has to be
//     cleared between calls (each call rewrites every partial it later reads),
//     but two calls that overlap on the GPU (for example on different
//     streams) race on it.  Serialise them.
std::size_t mla_decode_static_capacity();

void mla_decode_forward_static_cuda(
    __nv_bfloat16* output,
    float* logsumexp,
    const __nv_bfloat16* query,
    const __nv_bfloat16* paged_kv_cache,
    const int* block_table,
    const int* cache_lengths,
    int batch_size,
    int heads,
    int kv_rank,
    int rope_size,
    int page_size,
    int pages_per_sequence,
    int splits,
    float scale,
    cudaStream_t stream = nullptr);

// ---------------------------------------------------------------------------
// Non-absorbed causal prefill / training path (no counterpart in the reference).
//
// Dense layout (cu_seqlens == nullptr): q_nope [B,S,H,128], q_pe [B,S,H,64],
// k_nope [B,S,H,128], k_pe [B,S,1,64], v [B,S,H,128]; output [B,S,H,128],
// logsumexp [B,H,S].  Pass batch_size = B, max_sequence_length = S,
// total_tokens = B*S.
//
// Packed layout (cu_seqlens = device int32 [batch_size+1], cu_seqlens[0] = 0):
// the leading [B,S] of every tensor becomes [total_tokens]; attention is causal
// inside each sequence; logsumexp is [H,total_tokens].  Pass batch_size = number
// of sequences and max_sequence_length >= the longest sequence.
//
// q_pe and k_pe are taken as given (already rotated).  nope_size, rope_size and
// value_size must be 128, 64 and 128; scale must be positive.
// ---------------------------------------------------------------------------
void mla_prefill_forward_cuda(
    __nv_bfloat16* output,
    float* logsumexp,
    const __nv_bfloat16* q_nope,
    const __nv_bfloat16* q_pe,
    const __nv_bfloat16* k_nope,
    const __nv_bfloat16* k_pe,
    const __nv_bfloat16* v,
    const int* cu_seqlens,
    int batch_size,
    int max_sequence_length,
    int total_tokens,
    int heads,
    int nope_size,
    int rope_size,
    int value_size,
    float scale,
    cudaStream_t stream = nullptr);

// The backward runs as: key-side kernel (dK, dV, and dS^T of a group of heads left in the workspace), then
// dQ = dS K streamed from there, group after group; nothing is recomputed, at the price of workspace:
// 2 bytes per causal (query, key) pair and head of a group, in 128 x 64 tiles.  The workspace size is a
// bound that needs no lengths (every sequence at most max_sequence_length long, squares of the lengths
// at most max_sequence_length * total_tokens in sum); dense batches meet it exactly.  A group is as many
// heads as fit in the limit set here (default 20 GiB; the call returns the previous limit, a negative
// value only reads it).  When not even one head fits, dQ comes from a kernel that recomputes S and dP
// instead and the workspace is small.  Set the limit before asking for the workspace size and keep it
// unchanged until the backward call that uses that workspace.
std::size_t mla_prefill_backward_scratch_limit(long long bytes);

// Kernels one mla_prefill_backward_cuda call launches for this shape (`packed` is ignored: dense and
// packed batches take the same route).
int mla_prefill_backward_launches(int batch_size, int max_sequence_length, int total_tokens, int heads, bool packed);

// Bytes of caller-owned device scratch the backward needs.
std::size_t mla_prefill_backward_workspace_bytes(
    int batch_size,
    int max_sequence_length,
    int total_tokens,
    int heads);

// Backward of mla_prefill_forward_cuda.  Overwrites dq [..,H,192] (nope then
// pe), dk_nope [..,H,128], dk_pe [..,1,64] (summed over the heads of this call)
// and dv [..,H,128], all BF16.  The first total_tokens*64 FP32 values of the
// workspace hold the unrounded dk_pe sums afterwards, for callers that shard
// heads over several GPUs and add the partial sums themselves.  No output is
// accumulated with atomics (dk_pe adds the heads in index order), so two calls
// on the same inputs return the same bits.
void mla_prefill_backward_cuda(
    __nv_bfloat16* dq,
    __nv_bfloat16* dk_nope,
    __nv_bfloat16* dk_pe,
    __nv_bfloat16* dv,
    const __nv_bfloat16* output_gradient,
    const __nv_bfloat16* output,
    const float* logsumexp,
    const __nv_bfloat16* q_nope,
    const __nv_bfloat16* q_pe,
    const __nv_bfloat16* k_nope,
    const __nv_bfloat16* k_pe,
    const __nv_bfloat16* v,
    const int* cu_seqlens,
    void* workspace,
    int batch_size,
    int max_sequence_length,
    int total_tokens,
    int heads,
    int nope_size,
    int rope_size,
    int value_size,
    float scale,
    cudaStream_t stream = nullptr);

// No counterpart in the reference, which packs a whole [B,N,576] tensor into
// pages on the host (reference/python/mla.py:11-23).  Writes the rows of new
// tokens into the paged cache that mla_decode_forward_cuda reads: token t of
// sequence b goes to position start_positions[b] + t (0 when start_positions is
// null), i.e. page block_table[b][position / page_size], slot position %
// page_size, and the row is kv_latent[b,t,:] followed by key_rope[b,t,:].
//   kv_latent [B,T,512], key_rope [B,T,64] bf16; paged_kv_cache
//   [cache_blocks,page_size,1,576]; block_table [B,pages_per_sequence] int32;
//   token_counts [B] int32 or null: sequence b appends only its first
//   token_counts[b] of the T rows (ragged batches).
// A position past pages_per_sequence * page_size or a page number outside
// [0, cache_blocks) is not written and sets the device status to 3.
void mla_cache_append_cuda(
    __nv_bfloat16* paged_kv_cache,
    const __nv_bfloat16* kv_latent,
    const __nv_bfloat16* key_rope,
    const int* block_table,
    const int* start_positions,
    const int* token_counts,
    int batch_size,
    int tokens,
    int kv_rank,
    int rope_size,
    int page_size,
    int pages_per_sequence,
    int cache_blocks,
    cudaStream_t stream = nullptr);

// No counterpart in the reference (unquantised; reference/python/sources.json:2).  The cache in FP8:
// paged_fp8_cache is [cache_blocks, page_size, MLA_FP8_CACHE_ROW_BYTES] bytes, the row of a token being
// its 512 latent values as e4m3 (value = e4m3 * scale of its 128-column group), the four fp32 scales
// (max|x| of the group / 448, or 1 for a zero group) and its 64 rotary values in bf16.
// mla_cache_append_fp8_cuda quantises and writes the rows of new tokens, with the arguments, addressing
// and error behaviour of mla_cache_append_cuda.  mla_cache_dequantize_fp8_cuda rewrites the
// physical rows [first_row, first_row + rows) (row = page * page_size + slot) into a bf16 cache
// of the layout mla_decode_forward_cuda reads; decode over an FP8 cache is that pass followed by
// the bf16 decode.
void mla_cache_append_fp8_cuda(
    void* paged_fp8_cache,
    const __nv_bfloat16* kv_latent,
    const __nv_bfloat16* key_rope,
    const int* block_table,
    const int* start_positions,
    const int* token_counts,
    int batch_size,
    int tokens,
    int kv_rank,
    int rope_size,
    int page_size,
    int pages_per_sequence,
    int cache_blocks,
    cudaStream_t stream = nullptr);

void mla_cache_dequantize_fp8_cuda(
    __nv_bfloat16* paged_kv_cache,
    const void* paged_fp8_cache,
    long long first_row,
    long long rows,
    cudaStream_t stream = nullptr);

// No counterpart in the reference, whose benchmarks draw already-rotated inputs.
// Rotary position embedding, in place, of the 64 rotary columns the attention
// entry points take: q_pe [rows, heads, 64] and k_pe [rows, 1, 64] (either may be
// null).  Rotate-half pairing (element i with i + 32), angle = position *
// theta^(-2i/64).  positions [rows] int32 gives each row's position; when it is
// null the position is row % sequence_length (dense [B, S] rows).
void mla_rope_apply_cuda(
    __nv_bfloat16* q_pe,
    __nv_bfloat16* k_pe,
    const int* positions,
    long long rows,
    int heads,
    int sequence_length,
    int rope_size,
    float theta,
    cudaStream_t stream = nullptr);

// ---------------------------------------------------------------------------
// The dense projections either side of the attention kernels (no counterpart in
// the reference, whose benchmarks draw already-projected tensors).  W_UK and W_UV
// are the per-head up-projection weights stored [H*128, 512] (head h is rows
// [128h, 128h+128)); every tensor is bf16, row-major, contiguous; fp32 accumulate.
//
// mla_up_project_cuda: k_nope [rows, H, 128] = kv_latent [rows, 512] W_UK^T and
//   v [rows, H, 128] = kv_latent W_UV^T (either output may be null), the inputs
//   of mla_prefill_forward_cuda.
// mla_absorb_query_cuda: q_latent [rows, H, 512] = q_nope [rows, H, 128] W_UK[h],
//   the latent half of the query mla_decode_forward_cuda takes.
// mla_unabsorb_output_cuda: out [rows, H, 128] = o_latent [rows, H, 512] W_UV[h]^T,
//   applied to the decode output.
// ---------------------------------------------------------------------------
void mla_up_project_cuda(
    __nv_bfloat16* k_nope,
    __nv_bfloat16* v,
    const __nv_bfloat16* kv_latent,
    const __nv_bfloat16* w_uk,
    const __nv_bfloat16* w_uv,
    long long rows,
    int heads,
    cudaStream_t stream = nullptr);

void mla_absorb_query_cuda(
    __nv_bfloat16* q_latent,
    const __nv_bfloat16* q_nope,
    const __nv_bfloat16* w_uk,
    long long rows,
    int heads,
    cudaStream_t stream = nullptr);

void mla_unabsorb_output_cuda(
    __nv_bfloat16* output,
    const __nv_bfloat16* output_latent,
    const __nv_bfloat16* w_uv,
    long long rows,
    int heads,
    cudaStream_t stream = nullptr);

// Sticky device status shared by the kernels above: 0 = fine, 1 = a bounded
// pipeline wait inside a kernel ran out (results of that launch are invalid),
// 2 = a kernel found its shared memory misaligned, 3 = a cache append skipped (or
// a checked decode replaced) a page number or position outside the cache.
// Reading it synchronises the device; it is for tests and diagnosis, not for
// the hot path.  `reset` clears it after reading.
int mla_device_status(bool reset);

}  // namespace dscuda
