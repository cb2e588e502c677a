/* Provider ("params owner") host ABI, version 2 — the binary interface between a host broker
 * and the shared objects that fill a linked image's parameter blocks.
 *
 * This header restates the interface of the reference's
 * pipec/src/pipec2/host/include/pipelink_host_abi_v2.h so that a provider built against either
 * header loads under either broker: type names, field order, field widths, numeric codes and the
 * 0x700000xx type ids ARE the ABI and are therefore identical; everything else (wording, grouping,
 * helper names below the types) is this repository's.
 *
 * Rules of the interface (docs/reference/host-abi.md of the reference; pipec/README.md):
 *   - every top-level record starts with {abi_version = 2, struct_bytes};
 *   - only fixed-width integers, pointers and nested records cross it: no enum, bitfield,
 *     packed attribute or language-level tuple;
 *   - the broker allocates and owns every array and record; `query` fills demand arrays up to the
 *     stated capacities, `build` writes only residue[0, residue_cap) and its transfer reports and
 *     may create one private session that `release` frees exactly once;
 *   - addresses in resources are device addresses: a provider never dereferences them on the host;
 *   - return PLK_OK or one of PLK_E_*; nothing is thrown across the boundary.
 *
 * A provider for params group <s> exports exactly
 *   int pipelink_params_abi_<s>(plk_abi_report_v2*);
 *   int pipelink_params_query_<s>(const plk_common_v2*, const void* args, plk_demands_v2*);
 *   int pipelink_params_build_<s>(const plk_common_v2*, const void* args, const plk_resources_v2*,
 *                                 void* residue, size_t residue_cap, plk_transfer_report_v2*,
 *                                 uint32_t transfer_capacity, plk_session**);
 *   int pipelink_params_release_<s>(plk_session*);
 */
#ifndef PIPELINK_HOST_ABI_V2_H
#define PIPELINK_HOST_ABI_V2_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- numeric codes ------------------------------------------------------------------------ */
#define PLK_HOST_ABI_V2 2u

#define PLK_OK 0
#define PLK_E_VERSION 1  /* record version / size the callee does not speak */
#define PLK_E_CAPACITY 2 /* a broker-provided array is too small */
#define PLK_E_ARGUMENT 3 /* caller arguments are not acceptable */
#define PLK_E_CONTRACT 4 /* digests or declared channels do not match what was compiled in */
#define PLK_E_RESOURCE 5 /* a resource handed to build does not satisfy the demand */
#define PLK_E_BUILD 6    /* anything else that went wrong while building */
#define PLK_E_RELEASE 7

#define PLK_SCALAR_U64 1u
#define PLK_SCALAR_I64 2u
#define PLK_SCALAR_F64 3u
#define PLK_SCALAR_BOOL 4u

#define PLK_ACCESS_READ 1u
#define PLK_ACCESS_WRITE 2u
#define PLK_ACCESS_READ_WRITE 3u

/* How a transfer reported by `build` is represented inside the residue. */
#define PLK_TRANSFER_TMA_TILED 1u  /* a tiled tensor map (gather4 included) */
#define PLK_TRANSFER_TMA_IM2COL 2u /* an im2col tensor map */
#define PLK_TRANSFER_STRIDED 3u    /* a plain strided view, no encoder involved */

/* ---- small value records ------------------------------------------------------------------ */
typedef struct plk_header_v2 {
    uint32_t abi_version;
    uint32_t struct_bytes;
} plk_header_v2;

typedef struct plk_digest_v2 {
    uint8_t sha256[32];
} plk_digest_v2;

/* The profile facts an owner was compiled against: the dtype table's digest. */
typedef struct plk_profile_digest_v2 {
    plk_digest_v2 dtypes;
} plk_profile_digest_v2;

typedef struct plk_dim3_v2 {
    uint32_t x;
    uint32_t y;
    uint32_t z;
} plk_dim3_v2;

typedef struct plk_scalar_v2 {
    uint32_t scalar_id;
    uint32_t scalar_type; /* PLK_SCALAR_* */
    uint64_t value_bits;
} plk_scalar_v2;

/* A relocatable image: the records start record_offset bytes after this header. */
typedef struct plk_shared_scalars_v2 {
    plk_header_v2 header;
    uint64_t image_bytes;
    uint32_t record_count;
    uint32_t record_offset;
} plk_shared_scalars_v2;

/* What the caller says about a tensor at query time (no address yet). */
typedef struct plk_tensor_meta_v2 {
    uint32_t channel_id;
    uint32_t dtype_id;
    uint32_t rank;
    uint32_t access;
    uint64_t allocation_bytes;
    uint64_t alignment_bytes;
    uint64_t origin_byte_offset;
    uint32_t origin_bit_offset;
    uint32_t reserved;
    const uint64_t *extents;
    const int64_t *bit_strides;
} plk_tensor_meta_v2;

typedef struct plk_geometry_v2 {
    uint32_t geometry_present;
    uint32_t launch_required;
    plk_dim3_v2 grid;
    plk_dim3_v2 block;
    plk_dim3_v2 cluster;
    uint32_t reserved;
    uint64_t dynamic_smem_bytes;
} plk_geometry_v2;

/* One communication domain the owner declared by name ("ep", "tp", ...); rank and world are the
 * caller's facts for this session. */
typedef struct plk_domain_v2 {
    uint32_t domain_id;
    uint32_t rank;
    uint32_t world;
    uint32_t reserved;
} plk_domain_v2;

/* ---- what every call receives ------------------------------------------------------------- */
typedef struct plk_common_v2 {
    plk_header_v2 header;
    uint32_t owner_id;
    uint32_t channel_count;
    uint32_t domain_count;
    uint32_t reserved;
    const plk_shared_scalars_v2 *shared;
    const plk_tensor_meta_v2 *channels;
    const plk_domain_v2 *domains; /* ascending domain_id */
    plk_dim3_v2 block;
    plk_dim3_v2 cluster;
    uint64_t dynamic_smem_bytes;
    plk_profile_digest_v2 profile;
    plk_digest_v2 owner_contract;
} plk_common_v2;

/* ---- query: what the owner needs ---------------------------------------------------------- */
typedef struct plk_channel_demand_v2 {
    uint32_t channel_id;
    uint32_t dtype_id;
    uint32_t rank;
    uint32_t access;
    uint64_t minimum_allocation_bytes;
    uint64_t alignment_bytes;
    uint64_t *extents;    /* [rank], broker storage */
    int64_t *bit_strides; /* [rank], broker storage */
} plk_channel_demand_v2;

typedef struct plk_workspace_demand_v2 {
    uint32_t workspace_id;
    uint32_t reserved;
    uint64_t bytes;
    uint64_t alignment_bytes;
} plk_workspace_demand_v2;

typedef struct plk_demands_v2 {
    plk_header_v2 header;
    uint32_t channel_count;
    uint32_t channel_capacity;
    plk_channel_demand_v2 *channels;
    uint32_t workspace_count;
    uint32_t workspace_capacity;
    plk_workspace_demand_v2 *workspaces;
    plk_geometry_v2 geometry;
} plk_demands_v2;

/* ---- build: what the owner is given ------------------------------------------------------- */
/* A channel with a domain is one symmetric allocation per rank of that domain:
 * peer_addresses[r] is rank r's base as addressable from this rank (peer_addresses[own rank] ==
 * allocation_address), multicast_address the base in the domain's multicast window, 0 / NULL when
 * the channel declared no such view. */
typedef struct plk_device_resource_v2 {
    uint32_t channel_id;
    uint32_t access;
    uint64_t allocation_address;
    uint64_t allocation_bytes;
    uint64_t origin_byte_offset;
    uint32_t origin_bit_offset;
    uint32_t domain_id;
    const uint64_t *peer_addresses;
    uint64_t multicast_address;
} plk_device_resource_v2;

typedef struct plk_workspace_resource_v2 {
    uint32_t workspace_id;
    uint32_t reserved;
    uint64_t device_address;
    uint64_t bytes;
    uint64_t alignment_bytes;
} plk_workspace_resource_v2;

typedef struct plk_resources_v2 {
    plk_header_v2 header;
    uint32_t channel_count;
    uint32_t workspace_count;
    const plk_device_resource_v2 *channels;
    const plk_workspace_resource_v2 *workspaces;
    const plk_shared_scalars_v2 *shared;
    uint64_t cuda_stream_token;
    plk_geometry_v2 geometry;
} plk_resources_v2;

/* ---- build: what the owner reports back --------------------------------------------------- */
typedef struct plk_tma_tiled_detail_v2 {
    uint32_t swizzle; /* numeric CUtensorMapSwizzle */
    uint32_t rank;
    uint64_t box_elements[5];
    uint32_t element_strides[5];
    uint32_t reserved;
} plk_tma_tiled_detail_v2;

/* One record per declared transfer; the broker sets transfer_id and zeroes the rest. */
typedef struct plk_transfer_report_v2 {
    uint32_t transfer_id;
    uint32_t access;
    uint64_t residue_offset;       /* where the representation sits in this owner's residue */
    uint64_t representation_bytes; /* 128 for a tensor map */
    uint64_t representation_align;
    uint32_t storage_dtype_id;
    uint32_t ring_depth; /* 1 without a ring */
    uint64_t ring_stage_stride_bytes;
    uint64_t footprint_bytes_per_stage; /* bytes that land in this CTA's stage buffer */
    uint64_t credit_bytes_per_stage;    /* bytes credited to this CTA's completion barrier */
    uint64_t source_origin_bits;
    uint64_t source_span_bits;
    uint32_t vendor_kind; /* PLK_TRANSFER_* or 0 */
    uint32_t reserved;
    const void *vendor_detail; /* plk_tma_tiled_detail_v2 when vendor_kind is TMA_TILED */
} plk_transfer_report_v2;

/* ---- abi report: how this compiler laid the records out ------------------------------------ */
typedef struct plk_layout_entry_v2 {
    uint32_t abi_type_id;
    uint32_t reserved;
    uint64_t bytes;
    uint64_t alignment_bytes;
    plk_digest_v2 compiler_layout;
} plk_layout_entry_v2;

typedef struct plk_abi_report_v2 {
    plk_header_v2 header;
    uint32_t entry_count;
    uint32_t entry_capacity;
    plk_layout_entry_v2 *entries;
    plk_profile_digest_v2 profile;
    plk_digest_v2 owner_contract;
} plk_abi_report_v2;

/* Type ids of the records above (pipec-owned range 0x70000000 .. 0x700000ff). */
#define PLK_ABI_TYPE_ID_MIN 0x70000000u
#define PLK_ABI_TYPE_ID_MAX 0x700000ffu
enum {
    PLK_ABI_TYPE_ID_plk_abi_report_v2 = 0x70000001,
    PLK_ABI_TYPE_ID_plk_channel_demand_v2 = 0x70000002,
    PLK_ABI_TYPE_ID_plk_common_v2 = 0x70000003,
    PLK_ABI_TYPE_ID_plk_demands_v2 = 0x70000004,
    PLK_ABI_TYPE_ID_plk_tma_tiled_detail_v2 = 0x70000005,
    PLK_ABI_TYPE_ID_plk_device_resource_v2 = 0x70000006,
    PLK_ABI_TYPE_ID_plk_digest_v2 = 0x70000007,
    PLK_ABI_TYPE_ID_plk_dim3_v2 = 0x70000008,
    PLK_ABI_TYPE_ID_plk_geometry_v2 = 0x70000009,
    PLK_ABI_TYPE_ID_plk_header_v2 = 0x7000000a,
    PLK_ABI_TYPE_ID_plk_layout_entry_v2 = 0x7000000b,
    PLK_ABI_TYPE_ID_plk_profile_digest_v2 = 0x7000000c,
    PLK_ABI_TYPE_ID_plk_resources_v2 = 0x7000000d,
    PLK_ABI_TYPE_ID_plk_scalar_v2 = 0x7000000e,
    PLK_ABI_TYPE_ID_plk_shared_scalars_v2 = 0x7000000f,
    PLK_ABI_TYPE_ID_plk_transfer_report_v2 = 0x70000010,
    PLK_ABI_TYPE_ID_plk_tensor_meta_v2 = 0x70000011,
    PLK_ABI_TYPE_ID_plk_workspace_demand_v2 = 0x70000012,
    PLK_ABI_TYPE_ID_plk_workspace_resource_v2 = 0x70000013,
    PLK_ABI_TYPE_ID_plk_domain_v2 = 0x70000014
};
#define PLK_ABI_TYPE_ID(T) PLK_ABI_TYPE_ID_##T

/* One (id, size, alignment) row per record: what a provider's abi function reports. */
#ifdef __cplusplus
#define PLK_ALIGNOF(T) alignof(T)
#else
#define PLK_ALIGNOF(T) _Alignof(T)
#endif
#define PLK_LAYOUT_ROW(T) {PLK_ABI_TYPE_ID(T), 0u, sizeof(T), PLK_ALIGNOF(T), {{0}}}

/* The owner's declared domain with this id, or NULL. */
static inline const plk_domain_v2 *plk_find_domain(const plk_common_v2 *common, uint32_t domain_id) {
    uint32_t i;
    for (i = 0; i < common->domain_count; ++i)
        if (common->domains[i].domain_id == domain_id) return &common->domains[i];
    return NULL;
}

/* Provider-private bookkeeping; one per successful build. */
typedef struct plk_session_v2 plk_session;

typedef int (*plk_abi_fn_v2)(plk_abi_report_v2 *out);
typedef int (*plk_query_fn_v2)(const plk_common_v2 *common, const void *args, plk_demands_v2 *out);
typedef int (*plk_build_fn_v2)(const plk_common_v2 *common, const void *args,
                               const plk_resources_v2 *resources, void *residue, size_t residue_cap,
                               plk_transfer_report_v2 *transfers, uint32_t transfer_capacity,
                               plk_session **session);
typedef int (*plk_release_fn_v2)(plk_session *session);

#ifdef __cplusplus
}
#endif
#endif /* PIPELINK_HOST_ABI_V2_H */
