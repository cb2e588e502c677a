// A unit written for nothing but the annotation vocabulary: every declaration form of the annotation
// reference that the reference's shipped examples do not already exercise. It is packed by the
// reference's annotation pass (the record) and by this repo's header (the test); the two manifests
// must agree. Device bodies are empty on purpose.
#include <pipelink/stage.hpp>
#include <stdint.h>

struct VocabParams {
  const float* input;
  float* output;
  int32_t rows;
  int32_t cols;
};
struct alignas(128) VocabStorage {
  unsigned char bytes[4096];
};
struct VocabDescriptor {
  uint32_t opcode;
  uint32_t flags;
  uint64_t payload;
};

extern "C" __device__ int pipelink_vocab_depth();
extern "C" __device__ void vocab_feed(const void* params, unsigned variant) {}
extern "C" __device__ void vocab_drain(const void* params, unsigned variant) {}

PL_STAGE("org.vocab.unit", "2.1.0");
PL_PARAMS(VocabParams, input, output, rows, cols);
PL_ROLE(feed, vocab_feed, 1);
PL_ROLE(drain, vocab_drain, 4);
PL_DESCRIPTOR(VocabDescriptor);
PL_CLAIM_SMEM("pipelink_vocab_storage", VocabStorage, "kernel");
PL_CLAIM("pipelink_vocab_acc", "tmem", 128, 32, "kernel");
PL_CLAIM("pipelink_vocab_signal", "mbarrier", 1, 1, "kernel");
PL_CLAIM_EX(pl::claim("pipelink_vocab_ring", "smem").extent(256, {{"pipelink_vocab_depth", 8192}}).align(1024));
PL_CLAIM_EX(pl::claim("pipelink_vocab_full", "mbarrier").extent(0, {{"pipelink_vocab_depth", 1}}));
PL_CLAIM_EX(pl::claim("pipelink_vocab_empty", "mbarrier").extent(0, {{"pipelink_vocab_depth", 1}}));
PL_CLAIM_EX(pl::claim("pipelink_vocab_warp_feed", "warp").extent(1).roles({"feed"}));
PL_CLAIM_EX(pl::claim("pipelink_vocab_warp_drain", "warp").extent(4).align(4).roles({"drain"}));
PL_CLAIM("pipelink_vocab_flag", "gmem_counter", 2, 1, "kernel");
PL_ENDPOINT(tiles, pl::endpoint("tiles", pl::produce, "feed")
    .space("smem").scope("cta").proxy("async").tile("e4m3", {64, 128})
    .layout(pl::affine{{64, 128}, {128, 1}, 8}.swizzle(3, 4, 3))
    .protocol(pl::mbarrier{
        pl::side{"pipelink_vocab_full", pl::arrive{"feed", 1}, 8192},
        pl::side{"pipelink_vocab_empty", pl::arrive{"drain", "warps(drain)"}, 0},
        pl::init{"feed", 0, "dispatch"}})
    .ring(pl::handle("pipelink_vocab_depth"), 8192)
    .bind("base", "pipelink_vocab_ring")
    .bind("full", "pipelink_vocab_full")
    .bind("empty", "pipelink_vocab_empty"));
PL_ENDPOINT(acc, pl::endpoint("acc", pl::consume, "drain")
    .space("tmem").scope("cta").proxy("async").tile("f32", {128, 128})
    .layout(pl::tmem{0, 128, 128, 32})
    .protocol(pl::mbarrier{
        pl::side{"pipelink_vocab_signal", pl::arrive{"feed", 1}, 0},
        pl::side{"pipelink_vocab_signal", pl::arrive{"drain", "threads(drain)"}, 0},
        pl::init{"feed", 0, "dispatch"}})
    .ring(pl::fixed(1), 65536)
    .bind("base", "pipelink_vocab_acc"));
PL_ENDPOINT(done, pl::endpoint("done", pl::produce, "drain")
    .space("gmem").scope("system").proxy("generic").tile("u32", {1})
    .layout(pl::affine{{1}, {1}, 32})
    .protocol(pl::counter_sys{"pipelink_vocab_flag"}));
PL_ENDPOINT(ready, pl::endpoint("ready", pl::consume, "feed")
    .space("gmem").scope("grid").proxy("generic").tile("u32", {1})
    .layout(pl::affine{{1}, {1}, 32})
    .protocol(pl::counter{"pipelink_vocab_flag", "red.release.gpu", "ld.relaxed.gpu+fence.acquire.gpu"}));
PL_TOPOLOGY(pl::topology{2, pl::cluster{{2, 1, 1}, pl::launch{2, {8, 1, 1}}}, true, "static", {}});
PL_HINT("note", "vocabulary unit");
