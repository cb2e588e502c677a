/* A params provider with no device behind it, for tests of the host broker. The first 32-bit
 * word of `args` selects a misbehaviour; every call is appended to a log the test can read.
 * Group suffix: fake. Owner 1 states the geometry and declares one transfer on channel 1;
 * owner 2 asks for one workspace. Plain C against include/pipelink_host_abi_v2.h. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "pipelink_host_abi_v2.h"

enum { OK = 0, ABI_SIZE = 1, QUERY_ARGUMENT = 2, BUILD2_FAILS = 3, BUILD_MOVES_GEOMETRY = 4, TRANSFER_OUTSIDE = 5,
       DEMAND_TOO_BIG = 6, RELEASE1_FAILS = 7, TWO_GEOMETRIES = 8, WRONG_DEPTH = 9, NO_GEOMETRY = 10 };

static char g_log[1024];
static int g_live[8];

static void note(const char *what, unsigned owner) {
    char item[32];
    snprintf(item, sizeof item, "%s%u,", what, owner);
    strncat(g_log, item, sizeof g_log - strlen(g_log) - 1);
}
int fake_log(char *out, int cap) {
    strncpy(out, g_log, (size_t)cap - 1);
    out[cap - 1] = 0;
    return (int)strlen(g_log);
}
void fake_reset(void) {
    g_log[0] = 0;
    memset(g_live, 0, sizeof g_live);
}
static unsigned mode_of(const void *args) { return args ? *(const uint32_t *)args : 0; }

struct plk_session_v2 {
    unsigned owner;
};

int pipelink_params_abi_fake(plk_abi_report_v2 *out) {
    static const plk_layout_entry_v2 rows[] = {
        PLK_LAYOUT_ROW(plk_abi_report_v2), PLK_LAYOUT_ROW(plk_channel_demand_v2), PLK_LAYOUT_ROW(plk_common_v2),
        PLK_LAYOUT_ROW(plk_demands_v2), PLK_LAYOUT_ROW(plk_tma_tiled_detail_v2), PLK_LAYOUT_ROW(plk_device_resource_v2),
        PLK_LAYOUT_ROW(plk_digest_v2), PLK_LAYOUT_ROW(plk_dim3_v2), PLK_LAYOUT_ROW(plk_geometry_v2),
        PLK_LAYOUT_ROW(plk_header_v2), PLK_LAYOUT_ROW(plk_layout_entry_v2), PLK_LAYOUT_ROW(plk_profile_digest_v2),
        PLK_LAYOUT_ROW(plk_resources_v2), PLK_LAYOUT_ROW(plk_scalar_v2), PLK_LAYOUT_ROW(plk_shared_scalars_v2),
        PLK_LAYOUT_ROW(plk_transfer_report_v2), PLK_LAYOUT_ROW(plk_tensor_meta_v2), PLK_LAYOUT_ROW(plk_workspace_demand_v2),
        PLK_LAYOUT_ROW(plk_workspace_resource_v2), PLK_LAYOUT_ROW(plk_domain_v2)};
    uint32_t n = sizeof rows / sizeof rows[0];
    note("abi", 0);
    if (!out || out->header.abi_version != PLK_HOST_ABI_V2 || out->header.struct_bytes != sizeof *out) return PLK_E_VERSION;
    if (out->entry_capacity < n) return PLK_E_CAPACITY;
    memcpy(out->entries, rows, sizeof rows);
    if (getenv("FAKE_PROVIDER_ABI_SIZE")) out->entries[2].bytes += 8; /* pretend plk_common_v2 is laid out differently */
    out->entry_count = n;
    return PLK_OK;
}

int pipelink_params_query_fake(const plk_common_v2 *common, const void *args, plk_demands_v2 *out) {
    unsigned mode = mode_of(args);
    note("query", common->owner_id);
    if (mode == QUERY_ARGUMENT) return PLK_E_ARGUMENT;
    memset(&out->geometry, 0, sizeof out->geometry);
    out->channel_count = 0;
    out->workspace_count = 0;
    if (common->owner_id == 1) {
        plk_channel_demand_v2 *d = &out->channels[0];
        d->dtype_id = 1;
        d->access = PLK_ACCESS_READ;
        d->minimum_allocation_bytes = mode == DEMAND_TOO_BIG ? (1ull << 40) : 1024;
        d->alignment_bytes = 16;
        d->extents[0] = 1024;
        d->bit_strides[0] = 8;
        out->channel_count = 1;
    } else {
        out->workspaces[0].workspace_id = 7;
        out->workspaces[0].bytes = 4096;
        out->workspaces[0].alignment_bytes = 256;
        out->workspace_count = 1;
    }
    if ((common->owner_id == 1 && mode != NO_GEOMETRY) || (mode == TWO_GEOMETRIES)) {
        out->geometry.geometry_present = 1;
        out->geometry.launch_required = 1;
        out->geometry.grid.x = 3;
        out->geometry.grid.y = 2;
        out->geometry.grid.z = 1;
        out->geometry.block = common->block;
        out->geometry.cluster = common->cluster;
        out->geometry.dynamic_smem_bytes = common->dynamic_smem_bytes;
    }
    return PLK_OK;
}

int pipelink_params_build_fake(const plk_common_v2 *common, const void *args, const plk_resources_v2 *resources,
                               void *residue, size_t residue_cap, plk_transfer_report_v2 *transfers,
                               uint32_t transfer_capacity, plk_session **session) {
    unsigned mode = mode_of(args);
    static plk_tma_tiled_detail_v2 detail;
    note("build", common->owner_id);
    *session = NULL;
    if (common->owner_id == 2 && mode == BUILD2_FAILS) return PLK_E_BUILD;
    if (common->owner_id == 2 && (resources->workspace_count != 1 || resources->workspaces[0].bytes != 4096 ||
                                  resources->workspaces[0].device_address % 256 != 0))
        return PLK_E_RESOURCE;
    if (mode == BUILD_MOVES_GEOMETRY) ((plk_resources_v2 *)resources)->geometry.grid.x += 1;
    memset(residue, 0xA0 + (int)common->owner_id, residue_cap);
    if (common->owner_id == 1 && transfer_capacity >= 1) {
        plk_transfer_report_v2 *r = &transfers[0];
        r->access = PLK_ACCESS_READ;
        r->residue_offset = mode == TRANSFER_OUTSIDE ? residue_cap : 0;
        r->representation_bytes = 128;
        r->representation_align = 64;
        r->storage_dtype_id = 1;
        r->ring_depth = mode == WRONG_DEPTH ? 2 : 4;
        r->ring_stage_stride_bytes = 8192;
        r->footprint_bytes_per_stage = 8192;
        r->credit_bytes_per_stage = 8192;
        r->source_span_bits = 8192;
        r->vendor_kind = PLK_TRANSFER_TMA_TILED;
        r->vendor_detail = &detail;
    }
    *session = (plk_session *)malloc(sizeof(struct plk_session_v2));
    (*session)->owner = common->owner_id;
    g_live[common->owner_id] += 1;
    return PLK_OK;
}

int pipelink_params_release_fake(plk_session *session) {
    unsigned owner = session->owner;
    note("release", owner);
    g_live[owner] -= 1;
    free(session);
    return (owner == 1 && getenv("FAKE_PROVIDER_RELEASE1_FAILS")) ? PLK_E_RELEASE : PLK_OK;
}

int fake_live(unsigned owner) { return g_live[owner]; }
