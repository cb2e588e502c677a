// Expert-parallel plumbing over peer-mapped memory (NVLink / NVSwitch): symmetric
// allocation export/import, a flag barrier whose waits are bounded, the routes
// all-gather, and the dispatch pull of pre-quantised token rows.
//
// The reference exchanges token rows with comm CTAs that read peers' x_buffer and
// write peers' combine_buffer (campaigns/mok/port/comm/comm.cu:105-129,326-335) and
// brackets the kernel with barrier_all launches (campaigns/mok/host/mok_port_host.py:198-205).
// Here every rank quantises its own tokens once, peers pull E4M3 rows plus their scale
// words (half the NVLink bytes of pulling bf16, and bit-identical because MXFP8 blocks
// run along the hidden dimension of a single row), and the combine push happens inside
// the down GEMM's epilogue. Peer traffic is plain 16-byte loads and stores, except the
// default dispatch pull (ep_pull_rows_bulk_kernel), which reads rows from peers with untiled,
// non-multicast bulk copies (cp.async.bulk global -> shared). No copy with cluster multicast
// exists anywhere in this library.
//
// Counter protocol (examples/comm-overlap/comm/push_gather.cuh:16-150): flags are never
// reset; a launch generation kept in device memory gives each barrier its target value;
// signal = fence.acq_rel.sys + red.release.sys.add; wait = ld.acquire.sys with a
// wrap-safe signed compare and a cycle budget.
#include "kernels.h"

namespace plb {

namespace {

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* addr) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// One CTA. Thread i < world signals peer i's flag[rank] and waits for its own flag[i].
// state[0] is this rank's barrier generation (advanced by the kernel itself).
__global__ void ep_barrier_kernel(unsigned* const* flags_peers, unsigned* state, int rank, int world,
                                  Status* status) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  const unsigned target = state[0] + 1u;
  const int i = threadIdx.x;
  if (i < world) {
    fence_acq_rel_sys();
    red_release_sys_add(flags_peers[i] + rank, 1u);
    const unsigned* mine = flags_peers[rank] + i;
    const long long t0 = clock64();
    for (unsigned it = 0;; ++it) {
      const unsigned v = ld_acquire_sys(mine);
      if (static_cast<int>(v - target) >= 0) break;
      if ((it & 255u) == 255u) {
        if (clock64() - t0 > kWaitBudgetCycles) {
          report_failure(status, ST_TIMEOUT_COUNTER, 200 + i, v, target);
          failed = 1;
          break;
        }
        __nanosleep(64);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // advance even after a failure so later barriers compare against fresh targets
    state[0] = target;
    __threadfence();
  }
}

// dst_peers[p] + rank * count .. : this rank's slice of every peer's gather buffer.
__global__ void ep_publish_kernel(const uint4* __restrict__ src, int64_t vecs,
                                  uint4* const* dst_peers, int rank, int world) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int p = 0; p < world; ++p) {
    uint4* dst = dst_peers[p] + static_cast<int64_t>(rank) * vecs;
    for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < vecs;
         v += stride)
      dst[v] = src[v];
  }
}

// One warp per scheduled row: copy H bytes of E4M3 and H/128 scale words from the
// owning rank's quantised token buffer into this rank's routed buffers.
__global__ void __launch_bounds__(256)
ep_pull_rows_kernel(const uint8_t* const* __restrict__ xq_peers,
                    const uint8_t* const* __restrict__ xsc_peers, const int* __restrict__ peer_rank,
                    const int* __restrict__ peer_token_idx, const int* __restrict__ num_rows_dev,
                    int64_t capacity, int hidden, uint8_t* __restrict__ x_routed_fp8,
                    uint8_t* __restrict__ x_routed_sc) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  int64_t rows = *num_rows_dev;
  if (rows > capacity) rows = capacity;
  const int vec_per_row = hidden >> 4;
  const int col_blocks = hidden >> 7;
  for (int64_t p = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; p < rows;
       p += warps) {
    const int src_rank = peer_rank[p];
    uint4* dst = reinterpret_cast<uint4*>(x_routed_fp8 + p * hidden);
    const size_t dst_sc_row = static_cast<size_t>(p >> 7) * col_blocks * 512 + (p & 31) * 16 +
                              ((p & 127) >> 5) * 4;
    if (src_rank < 0) {
      for (int v = lane; v < vec_per_row; v += 32) dst[v] = make_uint4(0u, 0u, 0u, 0u);
      for (int c = lane; c < col_blocks; c += 32)
        *reinterpret_cast<uint32_t*>(x_routed_sc + dst_sc_row + static_cast<size_t>(c) * 512) = 0u;
      continue;
    }
    const int64_t t = peer_token_idx[p];
    const uint4* src = reinterpret_cast<const uint4*>(xq_peers[src_rank] + t * hidden);
    const uint8_t* src_sc = xsc_peers[src_rank] + static_cast<size_t>(t >> 7) * col_blocks * 512 +
                            (t & 31) * 16 + ((t & 127) >> 5) * 4;
    // loads first, then stores, so several NVLink reads are in flight per lane
    for (int v0 = 0; v0 < vec_per_row; v0 += 128) {
      uint4 tmp[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int v = v0 + u * 32 + lane;
        if (v < vec_per_row) tmp[u] = src[v];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int v = v0 + u * 32 + lane;
        if (v < vec_per_row) dst[v] = tmp[u];
      }
    }
    for (int c = lane; c < col_blocks; c += 32) {
      const uint32_t w = *reinterpret_cast<const uint32_t*>(src_sc + static_cast<size_t>(c) * 512);
      *reinterpret_cast<uint32_t*>(x_routed_sc + dst_sc_row + static_cast<size_t>(c) * 512) = w;
    }
  }
}

// Context-parallel K/V exchange: push this rank's 128-token K and V blocks into every
// consumer's gathered (global-order) buffers and publish one counter per block.
// Stand-in for kv_gather_role_gather (campaigns/attention/src/sm90/stage_kv_gather.cu:16-78)
// with the primitives of examples/comm-overlap/comm/push_gather.cuh:80-103: all lanes copy with
// 16-byte generic stores (loads batched before stores), then fence.acq_rel.sys and one
// red.release.sys on the consumer's counter. Zigzag ownership (campaigns/attention/README.md:222-228):
// rank r holds chunks r and 2W-1-r of 2W; the early chunk is needed by every rank, the late
// chunk only by ranks <= r (causality), so tasks are (block, consumer) pairs in that set,
// visited in descending global position (the blocks consumers wait for first).
__global__ void __launch_bounds__(256)
cp_push_kv_kernel(const uint4* __restrict__ k_local, const uint4* __restrict__ v_local,
                  int chunk_blocks, int vec_per_block, int rank, int world,
                  uint4* const* __restrict__ k_peers, uint4* const* __restrict__ v_peers,
                  unsigned* const* __restrict__ ready_peers) {
  // task order: late chunk (consumers 0..rank) first, then early chunk (all consumers)
  const int late_tasks = chunk_blocks * (rank + 1);
  const int total = late_tasks + chunk_blocks * world;
  for (int t = blockIdx.x; t < total; t += gridDim.x) {
    int local_block, consumer, global_block;
    if (t < late_tasks) {
      const int b = chunk_blocks - 1 - t / (rank + 1);  // descending position
      consumer = t % (rank + 1);
      local_block = chunk_blocks + b;
      global_block = (2 * world - 1 - rank) * chunk_blocks + b;
    } else {
      const int u = t - late_tasks;
      const int b = chunk_blocks - 1 - u / world;
      consumer = u % world;
      local_block = b;
      global_block = rank * chunk_blocks + b;
    }
    const uint4* ks = k_local + static_cast<size_t>(local_block) * vec_per_block;
    const uint4* vs = v_local + static_cast<size_t>(local_block) * vec_per_block;
    uint4* kd = k_peers[consumer] + static_cast<size_t>(global_block) * vec_per_block;
    uint4* vd = v_peers[consumer] + static_cast<size_t>(global_block) * vec_per_block;
    for (int i0 = threadIdx.x; i0 < vec_per_block; i0 += blockDim.x * 4) {
      uint4 a[4], b[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < vec_per_block) { a[u] = ks[i]; b[u] = vs[i]; }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < vec_per_block) { kd[i] = a[u]; vd[i] = b[u]; }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      fence_acq_rel_sys();
      red_release_sys_add(ready_peers[consumer] + global_block, 1u);
    }
    __syncthreads();
  }
}

// Dispatch pull on the bulk-copy engine: a warp streams rows peer -> shared memory -> local
// memory with untiled bulk copies (one 4 KB request per row and direction instead of 256 16-byte
// ones), three rows in flight per warp. The scale words of a row (one 4-byte word per 128
// columns, 512 bytes apart in the tensor-core layout) travel through registers, loaded when the
// row's copy is issued and stored when it lands.
// Scale words of each token gathered into one contiguous run: [tokens, hidden / 128] u32 next to the
// tensor-core layout (where a row's words sit 512 bytes apart), so that a peer fetches a row's
// scales with one 128-byte request instead of one 32-byte sector per word.
__global__ void __launch_bounds__(256)
scale_rows_kernel(const uint8_t* __restrict__ xsc, int64_t tokens, int col_blocks, uint32_t* __restrict__ out) {
  const int64_t total = tokens * col_blocks;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / col_blocks;
    const int c = static_cast<int>(i - t * col_blocks);
    out[i] = *reinterpret_cast<const uint32_t*>(xsc + static_cast<size_t>(t >> 7) * col_blocks * 512 +
                                                static_cast<size_t>(c) * 512 + (t & 31) * 16 + ((t & 127) >> 5) * 4);
  }
}

constexpr int kPullWarps = 4;
constexpr int kPullStages = 4;
constexpr int kPullAhead = kPullStages - 1;

__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

__global__ void __launch_bounds__(kPullWarps * 32)
ep_pull_rows_bulk_kernel(const uint8_t* const* __restrict__ xq_peers, const uint8_t* const* __restrict__ xsc_peers,
                         const int* __restrict__ peer_rank, const int* __restrict__ peer_token_idx,
                         const int* __restrict__ num_rows_dev, int64_t capacity, int hidden,
                         uint8_t* __restrict__ x_routed_fp8, uint8_t* __restrict__ x_routed_sc, int scale_rows,
                         Status* status) {
  extern __shared__ __align__(128) uint8_t pull_smem[];
  __shared__ uint64_t bars[kPullWarps][kPullStages];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    for (int s = 0; s < kPullStages; ++s) mbar_init(smem_u32(&bars[warp][s]), 1);
    fence_mbar_init();
  }
  __syncthreads();
  int64_t rows = *num_rows_dev;
  if (rows > capacity) rows = capacity;
  const int col_blocks = hidden >> 7;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * kPullWarps;
  const int64_t w0 = static_cast<int64_t>(blockIdx.x) * kPullWarps + warp;
  const int64_t n = w0 < rows ? (rows - w0 + warps - 1) / warps : 0;      // rows of this warp: w0 + i * warps
  const uint32_t ring = smem_u32(pull_smem) + static_cast<uint32_t>(warp) * kPullStages * hidden;
  uint32_t sc_word[kPullStages];
  bool live[kPullStages];
  uint32_t parity = 0;                                                      // bit s: phase of stage s
  bool ok = true;

  // issue row i into stage s: the bulk load, and this lane's scale word into a register
  auto issue = [&](int64_t i, int s) {
    const int64_t p = w0 + i * warps;
    const int src_rank = peer_rank[p];
    live[s] = src_rank >= 0;
    sc_word[s] = 0u;
    if (!live[s]) return;
    const int64_t t = peer_token_idx[p];
    if (lane == 0) {
      const uint32_t bar = smem_u32(&bars[warp][s]);
      mbar_arrive_expect_tx(bar, static_cast<uint32_t>(hidden));
      bulk_load(ring + static_cast<uint32_t>(s) * hidden, xq_peers[src_rank] + t * hidden, static_cast<uint32_t>(hidden), bar);
    }
    if (lane < col_blocks) {
      if (scale_rows) {
        sc_word[s] = reinterpret_cast<const uint32_t*>(xsc_peers[src_rank])[t * col_blocks + lane];
      } else {
        const uint8_t* src_sc = xsc_peers[src_rank] + static_cast<size_t>(t >> 7) * col_blocks * 512 + (t & 31) * 16 +
                                ((t & 127) >> 5) * 4;
        sc_word[s] = *reinterpret_cast<const uint32_t*>(src_sc + static_cast<size_t>(lane) * 512);
      }
    }
  };
  // retire row i from stage s: wait for the load, store the row and the scale word
  auto retire = [&](int64_t i, int s) {
    const int64_t p = w0 + i * warps;
    uint8_t* dst = x_routed_fp8 + p * hidden;
    if (live[s]) {
      if (lane == 0) {
        if (!mbar_wait(smem_u32(&bars[warp][s]), (parity >> s) & 1u, status, ST_TIMEOUT_FULL, 320 + s)) ok = false;
        if (ok) {
          fence_proxy_async_smem();
          bulk_store(dst, ring + static_cast<uint32_t>(s) * hidden, static_cast<uint32_t>(hidden));
        } else {
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      parity ^= 1u << s;
      ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
    } else {
      uint4* d = reinterpret_cast<uint4*>(dst);
      for (int v = lane; v < (hidden >> 4); v += 32) d[v] = make_uint4(0u, 0u, 0u, 0u);
      // every retired row commits one group, so "at most one group pending" always means
      // "everything but the latest row's store has been read out of shared memory"
      if (lane == 0) asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
    if (lane < col_blocks) {
      const size_t off = static_cast<size_t>(p >> 7) * col_blocks * 512 + (p & 31) * 16 + ((p & 127) >> 5) * 4;
      *reinterpret_cast<uint32_t*>(x_routed_sc + off + static_cast<size_t>(lane) * 512) = sc_word[s];
    }
  };

  for (int64_t i0 = 0; i0 < n + kPullAhead && ok; i0 += kPullStages) {
#pragma unroll
    for (int u = 0; u < kPullStages; ++u) {
      const int64_t i = i0 + u;                        // row issued now, into stage u
      const int64_t r = i - kPullAhead;                // row retired now, from stage (u + 1) % stages
      if (r >= 0 && r < n && ok) retire(r, (u + 1) % kPullStages);
      if (i < n && ok) {
        // stage u was last read by the store of row i - stages, committed at least one retire ago
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        __syncwarp();
        issue(i, u);
      }
    }
  }
  if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  __syncwarp();
}

// Receive streams for the combine push. Writing row p to `token * topk + slot` of its home rank
// scatters 8 KB rows over the whole combine buffer of every peer; measured on eight GPUs that costs
// 1.31 ms where the same bytes written in order cost 0.75 ms. Here every (source, home) pair gets a
// stream in the home rank's receive buffer: row p of this rank goes to position
// rank * stream_cap + (number of earlier rows with the same home), and the home rank learns where
// each (token, slot) landed through a 4-byte index written beside it.
// One CTA: the ranks are a running count per home over the schedule's row order.
__global__ void __launch_bounds__(1024)
ep_stream_rows_kernel(const int* __restrict__ peer_rank, const int* __restrict__ dest_row,
                      const int* __restrict__ num_rows_dev, int64_t capacity, int rank, int world,
                      int64_t stream_cap, int* __restrict__ stream_row, int* const* __restrict__ index_peers) {
  __shared__ int warp_count[32][32];   // [warp][home]
  __shared__ int base[32];             // rows already counted per home
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int64_t rows = *num_rows_dev;
  if (rows > capacity) rows = capacity;
  if (threadIdx.x < 32) base[threadIdx.x] = 0;
  __syncthreads();
  for (int64_t p0 = 0; p0 < rows; p0 += 1024) {
    const int64_t p = p0 + threadIdx.x;
    const int h = p < rows ? peer_rank[p] : -1;
    const unsigned same = __match_any_sync(0xFFFFFFFFu, h);
    const int before = __popc(same & ((1u << lane) - 1u));
    if (lane < world) warp_count[warp][lane] = 0;
    __syncwarp();
    if (h >= 0 && before == 0) warp_count[warp][h] = __popc(same);
    __syncthreads();
    int pos = -1;
    if (h >= 0) {
      int earlier = base[h];
      for (int w = 0; w < warp; ++w) earlier += warp_count[w][h];
      pos = earlier + before;
    }
    __syncthreads();
    if (threadIdx.x < world) {
      int add = 0;
      for (int w = 0; w < 32; ++w) add += warp_count[w][threadIdx.x];
      base[threadIdx.x] += add;
    }
    if (p < rows) {
      const int row = h >= 0 ? static_cast<int>(static_cast<int64_t>(rank) * stream_cap + pos) : -1;
      stream_row[p] = row;
      if (h >= 0) index_peers[h][dest_row[p]] = row;
    }
    __syncthreads();
  }
}

// All-gather push (examples/comm-overlap README, "AllGather protocol": a chunk is copied to one
// peer, every writing thread's stores are fenced at system scope, one release increment lands on
// the peer's row-block counter). A task is one part of one 256-row block for one consumer; a
// rank's blocks go first to the consumer whose GEMM reaches them first (it starts at its own
// rows and walks upward through the ranks). The task for consumer == rank copies nothing: the
// shard already sits in this rank's gathered buffer, only its counters advance.
__global__ void __launch_bounds__(256)
tp_push_rows_kernel(const uint4* __restrict__ src, int blocks, int vec_per_part, int parts, int rank, int world,
                    uint4* const* __restrict__ gather_peers, unsigned* const* __restrict__ ready_peers) {
  const int per_consumer = blocks * parts;
  const int total = per_consumer * world;
  for (int t = blockIdx.x; t < total; t += gridDim.x) {
    const int ci = t / per_consumer, r = t - ci * per_consumer;
    const int b = r / parts, part = r - b * parts;
    const int consumer = (rank - 1 - ci + 2 * world) % world;      // ci = world - 1 is this rank itself
    if (consumer != rank) {
      const size_t off = (static_cast<size_t>(b) * parts + part) * vec_per_part;
      const uint4* s = src + off;
      uint4* d = gather_peers[consumer] + static_cast<size_t>(rank) * blocks * parts * vec_per_part + off;
      for (int i0 = threadIdx.x; i0 < vec_per_part; i0 += blockDim.x * 4) {
        uint4 a[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u * blockDim.x;
          if (i < vec_per_part) a[u] = s[i];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u * blockDim.x;
          if (i < vec_per_part) d[i] = a[u];
        }
      }
      __threadfence_system();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      fence_acq_rel_sys();
      red_release_sys_add(ready_peers[consumer] + rank * blocks + b, 1u);
    }
    __syncthreads();
  }
}

}  // namespace

cudaError_t launch_tp_push_rows(const void* src, int blocks, int64_t block_bytes, int parts, int rank, int world,
                                void* const* gather_peers, unsigned* const* ready_peers, int ctas,
                                cudaStream_t stream) {
  if (blocks == 0) return cudaSuccess;
  tp_push_rows_kernel<<<ctas, 256, 0, stream>>>(static_cast<const uint4*>(src), blocks,
                                                static_cast<int>((block_bytes / parts) >> 4), parts, rank, world,
                                                reinterpret_cast<uint4* const*>(gather_peers), ready_peers);
  return cudaGetLastError();
}

cudaError_t launch_cp_push_kv(const void* k_local, const void* v_local, int chunk_blocks,
                              int64_t block_bytes, int rank, int world, void* const* k_peers,
                              void* const* v_peers, unsigned* const* ready_peers, int ctas,
                              cudaStream_t stream) {
  if (chunk_blocks == 0) return cudaSuccess;
  cp_push_kv_kernel<<<ctas, 256, 0, stream>>>(
      static_cast<const uint4*>(k_local), static_cast<const uint4*>(v_local), chunk_blocks,
      static_cast<int>(block_bytes >> 4), rank, world, reinterpret_cast<uint4* const*>(k_peers),
      reinterpret_cast<uint4* const*>(v_peers), ready_peers);
  return cudaGetLastError();
}

cudaError_t launch_ep_barrier(unsigned* const* flags_peers, unsigned* state, int rank, int world,
                              Status* status, cudaStream_t stream) {
  ep_barrier_kernel<<<1, 32, 0, stream>>>(flags_peers, state, rank, world, status);
  return cudaGetLastError();
}

cudaError_t launch_ep_publish(const void* src, int64_t bytes, void* const* dst_peers, int rank,
                              int world, cudaStream_t stream) {
  const int64_t vecs = bytes >> 4;
  if (vecs == 0) return cudaSuccess;
  int64_t blocks = (vecs + 255) / 256;
  if (blocks > 64) blocks = 64;
  ep_publish_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
      static_cast<const uint4*>(src), vecs, reinterpret_cast<uint4* const*>(dst_peers), rank, world);
  return cudaGetLastError();
}

cudaError_t launch_ep_pull_rows(const void* const* xq_peers, const void* const* xsc_peers,
                                const int* peer_rank, const int* peer_token_idx,
                                const int* num_rows_dev, int64_t capacity, int hidden,
                                void* x_routed_fp8, void* x_routed_sc, cudaStream_t stream) {
  if (capacity == 0) return cudaSuccess;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  ep_pull_rows_kernel<<<sms * 8, 256, 0, stream>>>(
      reinterpret_cast<const uint8_t* const*>(xq_peers),
      reinterpret_cast<const uint8_t* const*>(xsc_peers), peer_rank, peer_token_idx, num_rows_dev,
      capacity, hidden, static_cast<uint8_t*>(x_routed_fp8), static_cast<uint8_t*>(x_routed_sc));
  return cudaGetLastError();
}

cudaError_t launch_ep_pull_rows_bulk(const void* const* xq_peers, const void* const* xsc_peers, const int* peer_rank,
                                     const int* peer_token_idx, const int* num_rows_dev, int64_t capacity, int hidden,
                                     void* x_routed_fp8, void* x_routed_sc, int scale_rows, Status* status,
                                     cudaStream_t stream) {
  if (capacity == 0) return cudaSuccess;
  // one scale word per lane and 16-byte aligned bulk copies
  if (hidden > 4096 || hidden % 128) return cudaErrorInvalidValue;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int smem = kPullWarps * kPullStages * hidden;
  cudaError_t err = cudaFuncSetAttribute(ep_pull_rows_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (err != cudaSuccess) return err;
  ep_pull_rows_bulk_kernel<<<sms * 3, kPullWarps * 32, smem, stream>>>(
      reinterpret_cast<const uint8_t* const*>(xq_peers), reinterpret_cast<const uint8_t* const*>(xsc_peers), peer_rank,
      peer_token_idx, num_rows_dev, capacity, hidden, static_cast<uint8_t*>(x_routed_fp8),
      static_cast<uint8_t*>(x_routed_sc), scale_rows, status);
  return cudaGetLastError();
}

cudaError_t launch_scale_rows(const void* xsc, int64_t tokens, int hidden, void* out, cudaStream_t stream) {
  if (tokens == 0) return cudaSuccess;
  const int64_t total = tokens * (hidden >> 7);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 1184) blocks = 1184;
  scale_rows_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<const uint8_t*>(xsc), tokens, hidden >> 7,
                                                                  static_cast<uint32_t*>(out));
  return cudaGetLastError();
}

cudaError_t launch_ep_stream_rows(const int* peer_rank, const int* dest_row, const int* num_rows_dev, int64_t capacity,
                                  int rank, int world, int64_t stream_cap, int* stream_row, int* const* index_peers,
                                  cudaStream_t stream) {
  if (capacity == 0) return cudaSuccess;
  if (world < 1 || world > 32) return cudaErrorInvalidValue;
  ep_stream_rows_kernel<<<1, 1024, 0, stream>>>(peer_rank, dest_row, num_rows_dev, capacity, rank, world, stream_cap,
                                                stream_row, index_peers);
  return cudaGetLastError();
}

}  // namespace plb
