// Params provider of the three-stage MXFP8 GEMM: host code only. For each of the three owners
// (load, MMA, epilogue) it states what it needs from the caller's tensors (`query`) and writes
// the owner's parameter block into the residue the broker hands it (`build`), tensor maps
// included. Counterpart of the reference's examples/hopper-gemm-split/host/owner/provider.cpp
// and campaigns/mok/port/gemm/provider.cu, against the same ABI (pipelink_host_abi_v2.h).
//
// Group suffix: gemm3. Owners: 1 load, 2 mma, 3 epilogue. Channels (group-wide ids):
// 1 A e4m3 [M,K], 2 A scales, 3 B e4m3 [N,K], 4 B scales, 5 bias bf16 [N], 6 out bf16 [M,N].
// Shared scalar 1 (u64): the ring depth the link solved, echoed in the transfer reports.
// args: {u32 M, N, K, 0}. Nothing is thrown across the boundary and nothing on the device is
// dereferenced here.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>
#include <new>
#include <set>

#include "../../../../include/pipelink_host_abi_v2.h"
#include "../gemm3.cuh"

namespace {

enum : uint32_t { kOwnerLoad = 1, kOwnerMma = 2, kOwnerEpilogue = 3 };
enum : uint32_t { kChA = 1, kChASc = 2, kChB = 3, kChBSc = 4, kChBias = 5, kChOut = 6 };
enum : uint32_t { kDtypeE4m3 = 1, kDtypeUe8m0 = 2, kDtypeBf16 = 3 };
enum : uint32_t { kScalarDepth = 1 };

struct Args {
  uint32_t m, n, k, reserved;
};

struct Need {
  uint32_t channel, dtype, rank, access;
  uint64_t bytes, align;
  uint64_t extents[4];
  int64_t bit_strides[4];
};

// What each owner needs for a problem of M x N x K.
int needs_of(uint32_t owner, const Args& a, Need* out) {
  const uint64_t M = a.m, N = a.n, K = a.k;
  auto matrix = [](uint32_t ch, uint64_t rows, uint64_t cols) {
    Need n{ch, kDtypeE4m3, 2, PLK_ACCESS_READ, rows * cols, 16, {rows, cols}, {static_cast<int64_t>(cols) * 8, 8}};
    return n;
  };
  auto scales = [](uint32_t ch, uint64_t rows, uint64_t cols) {
    Need n{ch, kDtypeUe8m0, 4, PLK_ACCESS_READ, rows / 128 * (cols / 128) * 512, 16, {rows / 128, cols / 128, 32, 16},
           {static_cast<int64_t>(cols / 128) * 4096, 4096, 128, 8}};
    return n;
  };
  if (owner == kOwnerLoad) {
    out[0] = matrix(kChA, M, K);
    out[1] = scales(kChASc, M, K);
    out[2] = matrix(kChB, N, K);
    out[3] = scales(kChBSc, N, K);
    return 4;
  }
  if (owner == kOwnerEpilogue) {
    out[0] = Need{kChBias, kDtypeBf16, 1, PLK_ACCESS_READ, N * 2, 16, {N}, {16}};
    out[1] = Need{kChOut, kDtypeBf16, 2, PLK_ACCESS_WRITE, M * N * 2, 16, {M, N}, {static_cast<int64_t>(N) * 16, 16}};
    return 2;
  }
  return 0;
}

bool header_ok(const plk_header_v2& h, size_t bytes) {
  return h.abi_version == PLK_HOST_ABI_V2 && h.struct_bytes == bytes;
}
bool args_ok(const Args* a) {
  return a != nullptr && a->m != 0 && a->n != 0 && a->k != 0 && a->m % 128 == 0 && a->n % 128 == 0 && a->k % 128 == 0;
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [rows, k] u8 row-major, box 128 rows x 128 bytes, 128-byte swizzle.
bool encode_operand(CUtensorMap* map, uint64_t address, uint64_t rows, uint64_t k) {
  static EncodeTiled fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return false;
    fn = reinterpret_cast<EncodeTiled>(sym);
  }
  const cuuint64_t dims[2] = {k, rows};
  const cuuint64_t strides[1] = {k};
  const cuuint32_t box[2] = {128, 128};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, reinterpret_cast<void*>(address), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// One per successful build; holds what the transfer reports point to.
struct plk_session_v2 {
  uint32_t owner;
  plk_tma_tiled_detail_v2 details[2];
};

namespace {
std::mutex g_mutex;
std::set<plk_session_v2*> g_live;   // release must see a session exactly once

const plk_device_resource_v2* find_resource(const plk_resources_v2* r, uint32_t channel) {
  for (uint32_t i = 0; i < r->channel_count; ++i)
    if (r->channels[i].channel_id == channel) return &r->channels[i];
  return nullptr;
}
uint64_t shared_u64(const plk_shared_scalars_v2* s, uint32_t id, uint64_t fallback) {
  if (s == nullptr) return fallback;
  const plk_scalar_v2* rec = reinterpret_cast<const plk_scalar_v2*>(reinterpret_cast<const char*>(s) + s->record_offset);
  for (uint32_t i = 0; i < s->record_count; ++i)
    if (rec[i].scalar_id == id && rec[i].scalar_type == PLK_SCALAR_U64) return rec[i].value_bits;
  return fallback;
}
}  // namespace

extern "C" int pipelink_params_abi_gemm3(plk_abi_report_v2* out) {
  if (out == nullptr || !header_ok(out->header, sizeof(*out))) return PLK_E_VERSION;
  static const plk_layout_entry_v2 rows[] = {
      PLK_LAYOUT_ROW(plk_abi_report_v2),      PLK_LAYOUT_ROW(plk_channel_demand_v2),  PLK_LAYOUT_ROW(plk_common_v2),
      PLK_LAYOUT_ROW(plk_demands_v2),         PLK_LAYOUT_ROW(plk_tma_tiled_detail_v2), PLK_LAYOUT_ROW(plk_device_resource_v2),
      PLK_LAYOUT_ROW(plk_digest_v2),          PLK_LAYOUT_ROW(plk_dim3_v2),            PLK_LAYOUT_ROW(plk_geometry_v2),
      PLK_LAYOUT_ROW(plk_header_v2),          PLK_LAYOUT_ROW(plk_layout_entry_v2),    PLK_LAYOUT_ROW(plk_profile_digest_v2),
      PLK_LAYOUT_ROW(plk_resources_v2),       PLK_LAYOUT_ROW(plk_scalar_v2),          PLK_LAYOUT_ROW(plk_shared_scalars_v2),
      PLK_LAYOUT_ROW(plk_transfer_report_v2), PLK_LAYOUT_ROW(plk_tensor_meta_v2),     PLK_LAYOUT_ROW(plk_workspace_demand_v2),
      PLK_LAYOUT_ROW(plk_workspace_resource_v2), PLK_LAYOUT_ROW(plk_domain_v2)};
  const uint32_t n = sizeof(rows) / sizeof(rows[0]);
  if (out->entries == nullptr || out->entry_capacity < n) return PLK_E_CAPACITY;
  std::memcpy(out->entries, rows, sizeof(rows));
  out->entry_count = n;
  return PLK_OK;
}

extern "C" int pipelink_params_query_gemm3(const plk_common_v2* common, const void* raw_args, plk_demands_v2* out) {
  if (common == nullptr || out == nullptr || !header_ok(common->header, sizeof(*common)) ||
      !header_ok(out->header, sizeof(*out)))
    return PLK_E_VERSION;
  const Args* args = static_cast<const Args*>(raw_args);
  if (!args_ok(args)) return PLK_E_ARGUMENT;
  if (common->owner_id < kOwnerLoad || common->owner_id > kOwnerEpilogue) return PLK_E_CONTRACT;
  Need needs[4];
  const int n = needs_of(common->owner_id, *args, needs);
  if (out->channel_capacity < static_cast<uint32_t>(n)) return PLK_E_CAPACITY;
  for (int i = 0; i < n; ++i) {
    plk_channel_demand_v2& d = out->channels[i];
    // the broker initialised ids, ranks and the extents / strides storage from the declared channels
    if (d.channel_id != needs[i].channel || d.rank != needs[i].rank || d.extents == nullptr || d.bit_strides == nullptr)
      return PLK_E_CONTRACT;
    d.dtype_id = needs[i].dtype;
    d.access = needs[i].access;
    d.minimum_allocation_bytes = needs[i].bytes;
    d.alignment_bytes = needs[i].align;
    for (uint32_t r = 0; r < d.rank; ++r) {
      d.extents[r] = needs[i].extents[r];
      d.bit_strides[r] = needs[i].bit_strides[r];
    }
  }
  out->channel_count = static_cast<uint32_t>(n);
  out->workspace_count = 0;
  std::memset(&out->geometry, 0, sizeof(out->geometry));
  if (common->owner_id == kOwnerLoad) {   // the load owner is the launch-geometry authority
    out->geometry.geometry_present = 1;
    out->geometry.launch_required = 1;
    out->geometry.grid = plk_dim3_v2{args->m / 128, args->n / 128, 1};
    out->geometry.block = common->block;
    out->geometry.cluster = common->cluster;
    out->geometry.dynamic_smem_bytes = common->dynamic_smem_bytes;
  }
  return PLK_OK;
}

extern "C" int pipelink_params_build_gemm3(const plk_common_v2* common, const void* raw_args,
                                           const plk_resources_v2* resources, void* residue, size_t residue_cap,
                                           plk_transfer_report_v2* transfers, uint32_t transfer_capacity,
                                           plk_session** session) {
  if (common == nullptr || resources == nullptr || session == nullptr || !header_ok(common->header, sizeof(*common)) ||
      !header_ok(resources->header, sizeof(*resources)))
    return PLK_E_VERSION;
  *session = nullptr;
  const Args* args = static_cast<const Args*>(raw_args);
  if (!args_ok(args) || residue == nullptr) return PLK_E_ARGUMENT;
  Need needs[4];
  const int n = needs_of(common->owner_id, *args, needs);
  const plk_device_resource_v2* res[4] = {nullptr, nullptr, nullptr, nullptr};
  for (int i = 0; i < n; ++i) {
    res[i] = find_resource(resources, needs[i].channel);
    if (res[i] == nullptr) return PLK_E_CONTRACT;
    if (res[i]->allocation_bytes - res[i]->origin_byte_offset < needs[i].bytes ||
        (res[i]->allocation_address + res[i]->origin_byte_offset) % needs[i].align != 0 || res[i]->origin_bit_offset != 0)
      return PLK_E_RESOURCE;
  }
  auto address = [&](int i) { return res[i]->allocation_address + res[i]->origin_byte_offset; };
  plk_session_v2* s = new (std::nothrow) plk_session_v2();
  if (s == nullptr) return PLK_E_BUILD;
  s->owner = common->owner_id;
  int rc = PLK_OK;
  if (common->owner_id == kOwnerLoad) {
    if (residue_cap < sizeof(Gemm3LoadParams) || transfer_capacity < 2) {
      rc = PLK_E_CAPACITY;
    } else {
      Gemm3LoadParams p;
      std::memset(&p, 0, sizeof(p));
      if (!encode_operand(&p.a, address(0), args->m, args->k) || !encode_operand(&p.b, address(2), args->n, args->k)) {
        rc = PLK_E_BUILD;
      } else {
        p.a_sc = reinterpret_cast<const uint8_t*>(address(1));
        p.b_sc = reinterpret_cast<const uint8_t*>(address(3));
        p.K = static_cast<int>(args->k);
        std::memcpy(residue, &p, sizeof(p));
        const uint64_t depth = shared_u64(common->shared, kScalarDepth, 1);
        for (int t = 0; t < 2; ++t) {
          plk_tma_tiled_detail_v2& d = s->details[t];
          std::memset(&d, 0, sizeof(d));
          d.swizzle = static_cast<uint32_t>(CU_TENSOR_MAP_SWIZZLE_128B);
          d.rank = 2;
          d.box_elements[0] = 128;
          d.box_elements[1] = 128;
          d.element_strides[0] = d.element_strides[1] = 1;
          plk_transfer_report_v2& r = transfers[t];   // transfer_id was set by the broker
          r.access = PLK_ACCESS_READ;
          r.residue_offset = t == 0 ? offsetof(Gemm3LoadParams, a) : offsetof(Gemm3LoadParams, b);
          r.representation_bytes = sizeof(CUtensorMap);
          r.representation_align = 64;
          r.storage_dtype_id = kDtypeE4m3;
          r.ring_depth = static_cast<uint32_t>(depth);
          r.ring_stage_stride_bytes = gemm3::SlotBytes;
          r.footprint_bytes_per_stage = gemm3::OperandBytes;
          r.credit_bytes_per_stage = gemm3::OperandBytes;
          r.source_origin_bits = 0;
          r.source_span_bits = static_cast<uint64_t>(t == 0 ? args->m : args->n) * args->k * 8;
          r.vendor_kind = PLK_TRANSFER_TMA_TILED;
          r.vendor_detail = &d;
        }
      }
    }
  } else if (common->owner_id == kOwnerMma) {
    if (residue_cap < sizeof(Gemm3MmaParams)) {
      rc = PLK_E_CAPACITY;
    } else {
      Gemm3MmaParams p;
      std::memset(&p, 0, sizeof(p));
      p.K = static_cast<int>(args->k);
      std::memcpy(residue, &p, sizeof(p));
    }
  } else if (common->owner_id == kOwnerEpilogue) {
    if (residue_cap < sizeof(Gemm3EpilogueParams)) {
      rc = PLK_E_CAPACITY;
    } else {
      Gemm3EpilogueParams p;
      std::memset(&p, 0, sizeof(p));
      p.bias = reinterpret_cast<const void*>(address(0));
      p.out = reinterpret_cast<void*>(address(1));
      p.N = static_cast<int>(args->n);
      std::memcpy(residue, &p, sizeof(p));
    }
  } else {
    rc = PLK_E_CONTRACT;
  }
  if (rc != PLK_OK) {
    delete s;
    return rc;
  }
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_live.insert(s);
  }
  *session = s;
  return PLK_OK;
}

extern "C" int pipelink_params_release_gemm3(plk_session* session) {
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (session == nullptr || g_live.erase(session) == 0) return PLK_E_RELEASE;   // unknown or released twice
  }
  delete session;
  return PLK_OK;
}
