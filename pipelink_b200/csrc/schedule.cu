// Routing schedule: turns the all-gathered top-k expert ids of every rank into the
// padded, expert-sorted row list one rank's grouped GEMMs run over. It stands in for
// the reference's host-launched ops.schedule_out (campaigns/mok/host/mok_port_host.py:59-69),
// whose outputs are peer_rank / peer_token_idx / num_tokens / tokens_per_expert
// (compared bitwise there, :356-363) with every expert segment padded to
// EXPERT_PADDING rows and padding rows marked peer_rank = -1 (:93-96).
//
// Row order inside an expert segment is ascending (source rank, token, slot), i.e.
// ascending position in the gathered routes array. Three launches, no atomics on
// global memory, so the result is a pure function of the routes:
//   count : per 1024-entry chunk, per local expert, how many entries route to it
//   scan  : per expert exclusive scan over chunks, padded segment offsets,
//           block -> expert map, totals
//   fill  : per chunk, entries are ranked among same-expert entries with warp match masks
//           and per-warp counts, 256 entries per round, and written to their rows
#include "kernels.h"

namespace plb {

namespace {

__global__ void schedule_count_kernel(const int* __restrict__ routes, int64_t entries,
                                      int expert_base, int num_local_experts,
                                      int* __restrict__ chunk_counts) {
  extern __shared__ int hist[];
  for (int e = threadIdx.x; e < num_local_experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int64_t begin = static_cast<int64_t>(blockIdx.x) * kScheduleChunk;
  for (int i = threadIdx.x; i < kScheduleChunk; i += blockDim.x) {
    const int64_t idx = begin + i;
    if (idx < entries) {
      const int e = routes[idx] - expert_base;
      if (e >= 0 && e < num_local_experts) atomicAdd(&hist[e], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_local_experts; e += blockDim.x)
    chunk_counts[static_cast<int64_t>(blockIdx.x) * num_local_experts + e] = hist[e];
}

__global__ void schedule_scan_kernel(ScheduleArgs a, int chunks) {
  extern __shared__ int padded[];  // [num_local_experts + 1]
  const int E = a.num_local_experts;
  // one warp per expert (strided): lanes scan 32 chunks at a time with a running carry
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int e = warp; e < E; e += warps) {
    int carry = 0;
    for (int base = 0; base < chunks; base += 32) {
      const int c = base + lane;
      const int64_t at = static_cast<int64_t>(c) * E + e;
      const int n = c < chunks ? a.scratch[at] : 0;
      int incl = n;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(0xFFFFFFFFu, incl, d);
        if (lane >= d) incl += up;
      }
      if (c < chunks) a.scratch[at] = carry + incl - n;
      carry += __shfl_sync(0xFFFFFFFFu, incl, 31);
    }
    if (lane == 0) {
      a.tokens_per_expert[e] = carry;
      padded[e] = (carry + a.padding - 1) / a.padding * a.padding;
    }
  }
  __syncthreads();
  if (a.stream_row != nullptr && chunks > 0) {
    // Inside an expert segment the rows of source rank r form one run. Its first row (relative to
    // the segment) is the exclusive count at r's first chunk; the rows rank r has in the segments
    // of earlier experts are what precedes that run in r's receive stream.
    const int per_rank_chunks = chunks / a.world;
    int* base = a.stream_tables;
    int* start = a.stream_tables + a.world * E;
    for (int i = threadIdx.x; i < a.world * E; i += blockDim.x) {
      const int r = i / E, e = i - r * E;
      start[i] = a.scratch[static_cast<int64_t>(r) * per_rank_chunks * E + e];
    }
    __syncthreads();
    if (threadIdx.x < a.world) {
      const int r = threadIdx.x;
      int running = 0;
      for (int e = 0; e < E; ++e) {
        const int end = r + 1 < a.world ? start[(r + 1) * E + e] : a.tokens_per_expert[e];
        base[r * E + e] = running;
        running += end - start[r * E + e];
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    int64_t off = 0;
    for (int e = 0; e < E; ++e) {
      const int n = padded[e];
      padded[e] = static_cast<int>(off);
      off += n;
    }
    if (off > a.capacity) {
      report_failure(a.status, ST_BAD_ARGUMENT, 100, static_cast<unsigned>(off),
                     static_cast<unsigned>(a.capacity));
      // leave an empty schedule behind so downstream stages do nothing
      for (int e = 0; e <= E; ++e) padded[e] = 0;
      off = 0;
    }
    padded[E] = static_cast<int>(off);
    *a.num_tokens = static_cast<int>(off);
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) a.expert_offsets[e] = padded[e];
  const int blocks = a.capacity >> 7;
  for (int b = threadIdx.x; b < blocks; b += blockDim.x) {
    const int row = b << 7;
    int owner = -1;
    if (row < padded[E]) {
      int lo = 0, hi = E;  // last e with padded[e] <= row
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (padded[mid] <= row) lo = mid; else hi = mid;
      }
      owner = lo;
    }
    a.block_expert[b] = owner;
  }
}

// Stable placement of one 1024-entry chunk, 256 entries per round: an entry's row is
// (rows of its expert placed by earlier chunks and rounds) + (same-expert entries in
// earlier warps of this round) + (same-expert entries in earlier lanes of its warp).
// smem: run[E] running row per expert, wcnt[8][E] per-warp counts of the current round.
__global__ void __launch_bounds__(256)
schedule_fill_kernel(ScheduleArgs a, int64_t entries) {
  extern __shared__ int fill_smem[];
  const int E = a.num_local_experts;
  int* run = fill_smem;
  int* wcnt = fill_smem + E;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = a.expert_offsets[E];
  if (total == 0) return;  // empty (or overflowed) schedule: nothing to place
  const int64_t begin = static_cast<int64_t>(blockIdx.x) * kScheduleChunk;
  const int64_t per_rank = static_cast<int64_t>(a.tokens) * a.topk;
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    run[e] = a.expert_offsets[e] + a.scratch[static_cast<int64_t>(blockIdx.x) * E + e];
  for (int round = 0; round < kScheduleChunk / 256; ++round) {
    for (int i = threadIdx.x; i < 8 * E; i += blockDim.x) wcnt[i] = 0;
    __syncthreads();
    const int64_t idx = begin + round * 256 + threadIdx.x;
    int e = -1;
    if (idx < entries) {
      e = a.routes[idx] - a.expert_base;
      if (e < 0 || e >= E) e = -1;
    }
    const unsigned peers = __match_any_sync(0xFFFFFFFFu, e);
    const int before = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && before == 0) wcnt[warp * E + e] = __popc(peers);
    __syncthreads();
    if (e >= 0) {
      int pos = run[e] + before;
      for (int w = 0; w < warp; ++w) pos += wcnt[w * E + e];
      const int src = static_cast<int>(idx / per_rank);
      const int rem = static_cast<int>(idx - src * per_rank);
      a.peer_rank[pos] = src;
      a.peer_token_idx[pos] = rem / a.topk;
      a.dest_row[pos] = rem;
      if (a.stream_row != nullptr) {
        const int in_run = pos - a.expert_offsets[e] - a.stream_tables[(a.world + src) * E + e];
        const int at = static_cast<int>(static_cast<int64_t>(a.rank) * a.stream_cap) + a.stream_tables[src * E + e] + in_run;
        a.stream_row[pos] = at;
        a.stream_index_peers[src][rem] = at;
      }
    }
    __syncthreads();
    for (int x = threadIdx.x; x < E; x += blockDim.x) {
      int add = 0;
#pragma unroll
      for (int w = 0; w < 8; ++w) add += wcnt[w * E + x];
      run[x] += add;
    }
    __syncthreads();
  }
  if (blockIdx.x == 0) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      const int live_end = a.expert_offsets[e] + a.tokens_per_expert[e];
      const int seg_end = a.expert_offsets[e + 1];
      for (int p = live_end; p < seg_end; ++p) {
        a.peer_rank[p] = -1;
        a.peer_token_idx[p] = 0;
        a.dest_row[p] = -1;
        if (a.stream_row != nullptr) a.stream_row[p] = -1;
      }
    }
  }
}

// Scratch for launch_schedule_static: chunk counts for callers that hand over no
// workspace. 1 MiB, resident on every device that loads this library until the
// process exits. Its name is only a host-side handle here; the device address is
// looked up once per device below.
constexpr int64_t kStaticScratchInts = 262144;
static __device__ __align__(256) int g_schedule_scratch[kStaticScratchInts];

constexpr int kMaxDevices = 64;
int* g_static_scratch_ptr[kMaxDevices] = {};

}  // namespace

int64_t schedule_static_scratch_ints() { return kStaticScratchInts; }

cudaError_t launch_schedule_static(const ScheduleArgs& args, cudaStream_t stream) {
  const int64_t entries = static_cast<int64_t>(args.world) * args.tokens * args.topk;
  if (schedule_scratch_ints(entries, args.num_local_experts) > kStaticScratchInts)
    return cudaErrorInvalidValue;
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  if (g_static_scratch_ptr[dev] == nullptr) {
    // one-time set-up for this device (it is the current device): resolve the
    // device address of the array; host code must never pass the symbol itself
    int* ptr = nullptr;
    err = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_schedule_scratch);
    if (err != cudaSuccess) return err;
    if (ptr == nullptr) return cudaErrorInvalidSymbol;
    g_static_scratch_ptr[dev] = ptr;
  }
  ScheduleArgs a = args;
  a.scratch = g_static_scratch_ptr[dev];
  return launch_schedule(a, stream);
}

cudaError_t launch_schedule(const ScheduleArgs& a, cudaStream_t stream) {
  const int64_t entries = static_cast<int64_t>(a.world) * a.tokens * a.topk;
  if (a.stream_row != nullptr &&
      (a.stream_index_peers == nullptr || a.stream_tables == nullptr || a.world > 1024 ||
       (static_cast<int64_t>(a.tokens) * a.topk) % kScheduleChunk != 0))
    return cudaErrorInvalidValue;
  const int chunks = static_cast<int>((entries + kScheduleChunk - 1) / kScheduleChunk);
  const int E = a.num_local_experts;
  if (chunks > 0) {
    schedule_count_kernel<<<chunks, 256, E * sizeof(int), stream>>>(a.routes, entries,
                                                                    a.expert_base, E, a.scratch);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return err;
  }
  schedule_scan_kernel<<<1, 1024, (E + 1) * sizeof(int), stream>>>(a, chunks);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return err;
  if (chunks > 0) {
    schedule_fill_kernel<<<chunks, 256, 9 * E * sizeof(int), stream>>>(a, entries);
    err = cudaGetLastError();
  }
  return err;
}

}  // namespace plb
