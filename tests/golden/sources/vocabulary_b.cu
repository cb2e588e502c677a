// Second vocabulary unit: a one-shot tile barrier, a completion-only endpoint, register claims, variants,
// an exported callable with a role-less endpoint, absolute placement and a phase lifetime.
#include <pipelink/stage.hpp>
#include <stdint.h>
#include <optional>

struct VocabBParams {
  float* output;
  int32_t count;
};

extern "C" __device__ void vocab_b_main(const void* params, unsigned variant) {}
extern "C" __device__ void vocab_b_side(const void* params, unsigned variant) {}
extern "C" __device__ void org_vocab_b_main_wide(const void* params, unsigned variant) {}
extern "C" __device__ int vocab_b_poll(int slot) { return slot; }
extern "C" __device__ unsigned long long vocab_b_wide(const unsigned char* bytes, short s, long long v, double d, bool flag, unsigned u,
                                                    float* out, char c, unsigned short h, long l, unsigned long ul) { return 0; }

PL_STAGE("org.vocab.b", "0.3.0");
PL_PARAMS(VocabBParams, output, count);
PL_ROLE(main, vocab_b_main, 4);
PL_ROLE(side, vocab_b_side, 4);
PL_EXPORT(poll, vocab_b_poll);
PL_CALL(poll_channel, vocab_b_poll, pl::consume, "poll");
PL_EXPORT(wide, vocab_b_wide);
PL_CALL(wide_channel, vocab_b_wide, pl::consume, "wide");
PL_CLAIM_REGS("pipelink_vocab_b_regs_main", "main", {232, 200, 168}, "main");
PL_CLAIM_REGS("pipelink_vocab_b_regs_side", "side", {40, 56}, "side");
PL_CLAIM_EX(pl::claim("pipelink_vocab_b_warp_main", "warp").extent(4).align(4).at(0).roles({"main"}));
PL_CLAIM_EX(pl::claim("pipelink_vocab_b_warp_side", "warp").extent(4).align(4).at(4).roles({"side"}));
PL_CLAIM_EX(pl::claim("pipelink_vocab_b_scratch", "smem").extent(2048).align(128).lifetime("phase:drain"));
PL_CLAIM("pipelink_vocab_b_a_full", "mbarrier", 1, 1, "kernel");
PL_CLAIM("pipelink_vocab_b_sig", "mbarrier", 2, 1, "kernel");
PL_CLAIM("pipelink_vocab_b_slot", "gmem_counter", 1, 1, "kernel");
PL_CLAIM("pipelink_vocab_b_tiles", "smem", 16384, 1024, "kernel");
PL_ENDPOINT(a_tiles, pl::endpoint("a_tiles", pl::produce, "main")
    .space("smem").scope("cta").proxy("async").tile("bf16", {64, 64})
    .layout(pl::affine{{64, 64}, {64, 1}, 16}.swizzle(3, 4, 3))
    .protocol(pl::mbarrier{
        pl::side{"pipelink_vocab_b_a_full", pl::arrive{"main", 1}, pl::tile},
        std::nullopt, pl::init{"main", 0, "stage"}, "never"})
    .ring(pl::fixed(1), 8192)
    .bind("base", "pipelink_vocab_b_tiles")
    .bind("full", "pipelink_vocab_b_a_full"));
PL_ENDPOINT(finished, pl::signal_endpoint("finished", pl::produce, "main")
    .scope("cluster")
    .protocol(pl::mbarrier{
        pl::side{"pipelink_vocab_b_sig", {"main", 2}, 0},
        std::nullopt, {"main", 0, "dispatch"}, "external"})
    .ring(pl::fixed(2), 0)
    .bind("full", "pipelink_vocab_b_sig"));
PL_ENDPOINT(progress, pl::endpoint("progress", pl::consume)
    .space("gmem").scope("grid").proxy("generic").tile("u32", {1})
    .layout(pl::affine{{1}, {1}, 32})
    .protocol(pl::counter{"pipelink_vocab_b_slot"})
    .exports({"poll"}));
PL_VARIANT(0, {{"pipelink_vocab_b_regs_main", 232}});
PL_VARIANT_ENTRY(1, {{"pipelink_vocab_b_regs_main", 200}}, org_vocab_b_main_wide);
PL_VARIANT(2, {{"pipelink_vocab_b_regs_main", 168}});
PL_TOPOLOGY(pl::topology{1, pl::cluster{{2, 1, 1}, pl::launch{2, {2, 1, 1}}}, false, "static", {}});
