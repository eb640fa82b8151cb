#include "plan_spec.h"

#include <algorithm>
#include <stdexcept>

namespace tmb {

namespace {

std::string Sources(std::initializer_list<std::string> names) {
  std::string out = "[";
  bool first = true;
  for (const auto& name : names) {
    if (!first) out += ',';
    out += Json::Quote(name);
    first = false;
  }
  return out + "]";
}

// "shard": the loader narrows every checkpoint tensor the recipe names to this rank's
// contiguous part on `axis` before the transform (python/tilemega/serving/weights.py:78-96).
std::string Shard(int axis, int parts) {
  if (parts < 2) return "";
  return ",\"shard\":{\"axis\":" + std::to_string(axis) + ",\"parts\":" + std::to_string(parts) + "}";
}

std::string Alias(const std::string& fqn, const std::string& shard = "") {
  return "{\"kind\":\"alias\",\"source\":" + Json::Quote(fqn) + shard + "}";
}

// The reference's tile_pages recipe (python/tilemega/serving/weights.py:204-242):
// [N/tile_n][K/tile_k][tile_n*tile_k] with the 8x64 128-byte XOR swizzle.
std::string Pages(const std::string& source, int tile_k, int tile_n = kTileN) {
  return "{\"kind\":\"tile_pages\",\"tile_n\":" + std::to_string(tile_n) + ",\"tile_k\":" + std::to_string(tile_k) +
         ",\"source\":" + source + "}";
}

// Dense-batch GEMM stage: row tiles of 128, the reduction in 128-column chunks cut into the fewest parts
// that give tasks to at least 85 % of the SMs (a part keeps at least four chunks, 128 KB of weights). Few
// parts matter: the last arriver of a tile reads every part's fp32 tile back, nsplit * batch loads per
// thread (measured at batch 64: 8 and 14 parts cost the QKV and down stages 3-4 times their streaming time).
DenseGeo MakeDenseGeo(const char* what, int n, int k, int sms) {
  if (n <= 0 || n % kDenseTileN) throw std::invalid_argument(std::string(what) + ": rows must be a multiple of 128 for a dense-batch plan");
  if (k <= 0 || k % kDenseTileK) throw std::invalid_argument(std::string(what) + ": K must be a multiple of 128 for a dense-batch plan");
  DenseGeo g{};
  g.n = n;
  g.k = k;
  g.tiles = n / kDenseTileN;
  const int chunks = k / kDenseTileK;
  g.nsplit = 1;
  for (int d = 1; d <= chunks; ++d) {
    if (chunks % d || chunks / d < std::min(4, chunks)) continue;
    g.nsplit = d;
    if (g.tiles * d * 20 >= sms * 17) break;   // tasks for at least 85 % of the SMs
  }
  g.cps = chunks / g.nsplit;
  g.ntasks = g.tiles * g.nsplit;
  if (g.ntasks >= 0xFFFF) throw std::invalid_argument(std::string(what) + ": too many tasks for the task FIFO's 16-bit ids");
  return g;
}

// The page stream of a dense-batch stage in the streaming thread's terms: a task is cps consecutive
// 32 KB pages of 128 rows x 128 columns.
GemvGeo StreamGeo(const DenseGeo& d) {
  GemvGeo g{};
  g.n = d.n;
  g.k = g.k_src = d.k;
  g.tile_k = kDenseTileK;
  g.pages_per_task = g.task_pages = d.cps;
  g.last_page_bytes = g.page_bytes = kSlotBytes;
  g.ntasks = d.ntasks;
  g.page0 = 0;
  g.src_off = 0;
  g.src_stride = d.k;
  g.claim_chunk = std::max(1, 65536 / (d.cps * kSlotBytes));
  return g;
}

// A reduction length that is not a multiple of the page width is rounded up: the
// tile_pages recipe zero-fills the weights' missing columns and the kernel zero-fills the
// activation rows', so the extra columns add nothing. Inside a page a 64-column block of
// the 8 rows is contiguous (1 KB), so the pad is the page's tail: the kernel copies only
// last_page_bytes of a task's last page and the pad costs address space, not bandwidth.
GemvGeo MakeGeo(const char* what, int n, int k, const Json& overrides, int elem_bytes = 2) {
  GemvGeo g{};
  g.n = n;
  g.k_src = k;
  g.tile_k = kSlotBytes / (kTileN * elem_bytes);   // 2048 columns of bf16, 4096 of e4m3: a page is one 32 KB slot
  if (k > 0 && k % 8 == 0) k = (k + g.tile_k - 1) / g.tile_k * g.tile_k;
  g.k = k;
  if (n <= 0 || n % kTileN) throw std::invalid_argument(std::string(what) + ": rows must be a multiple of 8");
  if (k <= 0 || k % g.tile_k) throw std::invalid_argument(std::string(what) + ": K must be a multiple of 8");
  const int kt = k / g.tile_k;
  g.pages_per_task = kt;
  // columns of the last page that hold weights, in whole warp shares (an eighth of a page)
  const int share = g.tile_k / 8;
  const int last_columns = (g.k_src - (kt - 1) * g.tile_k + share - 1) / share * share;
  g.last_page_bytes = kTileN * last_columns * elem_bytes;
  g.page_bytes = kSlotBytes;
  g.ntasks = n / kTileN;
  g.page0 = 0;
  g.task_pages = kt;
  g.src_off = 0;
  g.src_stride = g.k_src;
  const int task_bytes = (kt - 1) * g.page_bytes + g.last_page_bytes;
  g.claim_chunk = std::max(1, std::min(8, (65536 + task_bytes - 1) / task_bytes));
  if (overrides.has(what)) g.claim_chunk = int(overrides.at(what).integer("claim_chunk", g.claim_chunk));
  if (g.claim_chunk < 1 || g.claim_chunk > 64) throw std::invalid_argument(std::string(what) + ": claim_chunk must lie in [1, 64]");
  return g;
}

// A forward plan's table (the reference's forward runtime exposes the exported module's parameters under their
// qualified names, its int64 inputs and its outputs: include/tilemega/Codegen/tasks/Sm90F3Runtime.cuh:95-131,
// python/tilemega/dnn/check.py:33-66): the BertModel parameters in nn.Linear layout as they are (no packing: the
// GEMM kernel reads K-major rows through tensor maps), two int64 inputs, two outputs, four internal activations.
PlanSpec ForwardSpec(const Json& plan) {
  PlanSpec s;
  s.forward = true;
  const Json& model = plan.at("model");
  s.hidden = int(model.integer("hidden_size", 0));
  s.inter = int(model.integer("intermediate_size", 0));
  s.heads = int(model.integer("num_attention_heads", 0));
  s.layers = int(model.integer("num_hidden_layers", 0));
  s.vocab = int(model.integer("vocab_size", 0));
  s.max_position = int(model.integer("max_position_embeddings", 0));
  s.type_vocab = int(model.integer("type_vocab_size", 0));
  s.eps = model.num("layer_norm_eps", 1e-12);
  s.kv_heads = s.heads;
  s.head_dim = s.heads ? s.hidden / s.heads : 0;
  s.forward_seq = int(plan.integer("seq", 0));
  s.batch_lo = int(plan.integer("batch_lo", 1));
  s.batch_hi = int(plan.integer("batch_hi", s.batch_lo));
  s.grid = int(plan.integer("grid", 0));
  const std::string dtype = plan.str("dtype", "f16");
  if (dtype != "f16" && dtype != "bf16") throw std::invalid_argument("a forward plan computes in f16 or bf16 (dtype)");
  s.f16 = dtype == "f16";
  s.forward_mask = plan.flag("mask", false);
  if (model.str("hidden_act", "gelu") != "gelu") throw std::invalid_argument("the encoder's feed-forward is built with the erf GELU only");
  if (model.str("position_embedding_type", "absolute") != "absolute")
    throw std::invalid_argument("the encoder is built with absolute position embeddings only");
  if (s.hidden <= 0 || s.inter <= 0 || s.heads <= 0 || s.layers <= 0 || s.vocab <= 0 || s.type_vocab <= 0)
    throw std::invalid_argument("model dimensions must be positive");
  if (s.head_dim != 64 || s.heads * 64 != s.hidden) throw std::invalid_argument("encoder heads must be 64 wide");
  if (s.hidden % 128 || s.hidden > 1024) throw std::invalid_argument("encoder hidden size must be a multiple of 128, at most 1024");
  if (s.inter % 128) throw std::invalid_argument("encoder intermediate size must be a multiple of 128");
  if (s.forward_seq != 128 || s.forward_seq > s.max_position) throw std::invalid_argument("forward plans run sequences of 128 positions (seq)");
  if (s.batch_lo < 1 || s.batch_hi < s.batch_lo || s.batch_hi > 512) throw std::invalid_argument("forward batch interval must lie in [1, 512]");
  const uint32_t elem = s.f16 ? 5u : 0u;
  auto add = [&](const std::string& name, uint32_t role, uint32_t dtype, uint64_t constant, uint64_t per_batch, bool weight) {
    BufferSpec b;
    b.name = name;
    b.role = role;
    b.dtype = dtype;
    b.elements_constant = constant;
    b.elements_per_batch = per_batch;
    if (weight) b.pack_json = Alias(name);
    s.buffers.push_back(b);
  };
  const uint64_t H = uint64_t(s.hidden), I = uint64_t(s.inter), S = uint64_t(s.forward_seq);
  add("embeddings.word_embeddings.weight", 1, elem, uint64_t(s.vocab) * H, 0, true);
  add("embeddings.position_embeddings.weight", 1, elem, uint64_t(s.max_position) * H, 0, true);
  add("embeddings.token_type_embeddings.weight", 1, elem, uint64_t(s.type_vocab) * H, 0, true);
  add("embeddings.LayerNorm.weight", 1, elem, H, 0, true);
  add("embeddings.LayerNorm.bias", 1, elem, H, 0, true);
  for (int l = 0; l < s.layers; ++l) {
    const std::string p = "encoder.layer." + std::to_string(l) + ".";
    for (const char* part : {"query", "key", "value"}) {
      add(p + "attention.self." + part + ".weight", 1, elem, H * H, 0, true);
      add(p + "attention.self." + part + ".bias", 1, elem, H, 0, true);
    }
    add(p + "attention.output.dense.weight", 1, elem, H * H, 0, true);
    add(p + "attention.output.dense.bias", 1, elem, H, 0, true);
    add(p + "attention.output.LayerNorm.weight", 1, elem, H, 0, true);
    add(p + "attention.output.LayerNorm.bias", 1, elem, H, 0, true);
    add(p + "intermediate.dense.weight", 1, elem, I * H, 0, true);
    add(p + "intermediate.dense.bias", 1, elem, I, 0, true);
    add(p + "output.dense.weight", 1, elem, H * I, 0, true);
    add(p + "output.dense.bias", 1, elem, H, 0, true);
    add(p + "output.LayerNorm.weight", 1, elem, H, 0, true);
    add(p + "output.LayerNorm.bias", 1, elem, H, 0, true);
  }
  add("pooler.dense.weight", 1, elem, H * H, 0, true);
  add("pooler.dense.bias", 1, elem, H, 0, true);
  add("input_ids", 1, 3, 0, S, false);
  add("token_type_ids", 1, 3, 0, S, false);
  if (s.forward_mask) add("attention_mask", 1, 3, 0, S, false);
  add("last_hidden_state", 1, elem, 0, S * H, false);
  add("pooler_output", 1, elem, 0, H, false);
  add("forward.hidden", 0, elem, 0, S * H, false);
  add("forward.qkv", 0, elem, 0, S * 3 * H, false);
  add("forward.context", 0, elem, 0, S * H, false);
  add("forward.ffn", 0, elem, 0, S * I, false);
  return s;
}

}  // namespace

int PlanSpec::max_k() const {
  int widest = 0;
  for (int s = 0; s < kNumGemv; ++s)
    widest = std::max(widest, s == kDown && down_splits > 1 ? down_part[0].k : geo[s].k);   // columns staged at once
  return widest;
}

uint64_t PlanSpec::weight_bytes() const {
  uint64_t total = 0;
  for (int s = 0; s < kNumGemv; ++s) {
    uint64_t one = fp8 ? uint64_t(geo[s].n) * uint64_t(geo[s].k_src) + 4ull * uint64_t(geo[s].n)   // bytes + a scale per row
                       : 2ull * uint64_t(geo[s].n) * uint64_t(geo[s].k_src);
    if (experts && (s == kGateUp || s == kDown)) one *= uint64_t(topk) * uint64_t(batch_hi);   // experts routed to per step
    total += s == kHead ? one : one * uint64_t(layers);
  }
  return total;
}

PlanSpec PlanSpec::FromJson(const Json& plan) {
  PlanSpec s;
  const std::string phase = plan.str("phase", "decode");
  if (phase == "forward") return ForwardSpec(plan);
  if (phase != "decode" && phase != "prefill") throw std::invalid_argument("decode, prefill and forward plans are built (phase)");
  s.prefill = phase == "prefill";
  const Json& model = plan.at("model");
  s.hidden = int(model.integer("hidden_size", 0));
  s.inter = int(model.integer("intermediate_size", 0));
  s.heads = int(model.integer("num_attention_heads", 0));
  s.kv_heads = int(model.integer("num_key_value_heads", 0));
  s.layers = int(model.integer("num_hidden_layers", 0));
  s.vocab = int(model.integer("vocab_size", 0));
  s.head_dim = int(model.integer("head_dim", s.heads ? s.hidden / s.heads : 0));
  s.eps = model.num("rms_norm_eps", 1e-5);
  s.tied = model.flag("tie_word_embeddings", false);
  // mixture of experts (python/tilemega/moe/export.py:54-93): top-k of a softmax router,
  // expert SwiGLU FFNs of moe_intermediate_size; Qwen3 also normalises every q/k head
  s.experts = int(model.integer("num_experts", 0));
  if (s.experts) {
    s.topk = int(model.integer("num_experts_per_tok", 0));
    s.norm_topk = model.flag("norm_topk_prob", false);
    s.inter = int(model.integer("moe_intermediate_size", s.inter));
    if (s.experts % kTileN || s.experts > 256) throw std::invalid_argument("experts must be a multiple of 8, at most 256");
    if (s.topk < 1 || s.topk > kMaxTopK || s.topk > s.experts) throw std::invalid_argument("experts per token must lie in [1, 8]");
    if (!s.norm_topk) throw std::invalid_argument("only renormalised top-k routing (norm_topk_prob) is built");
  }
  if (model.has("architectures")) {
    const Json& arch = model.at("architectures");
    s.qk_norm = arch.kind == Json::kArray && !arch.items.empty() && arch.items[0].kind == Json::kString &&
                arch.items[0].text.rfind("Qwen3", 0) == 0;
  }
  if (s.hidden <= 0 || s.inter <= 0 || s.heads <= 0 || s.kv_heads <= 0 || s.layers <= 0 || s.vocab <= 0)
    throw std::invalid_argument("model dimensions must be positive");
  if (s.head_dim != 64 && s.head_dim != 128) throw std::invalid_argument("head_dim must be 64 or 128");
  if (s.heads % s.kv_heads || (s.heads / s.kv_heads != 4 && s.heads / s.kv_heads != 8))
    throw std::invalid_argument("query heads per KV head must be 4 or 8");
  if (s.heads / s.kv_heads == 8 && s.head_dim != 128)
    throw std::invalid_argument("8 query heads per KV head are built for head_dim 128 only");
  // tensor parallelism: every split dimension must divide (export.py:182-192)
  s.tp = int(plan.integer("tp", 1));
  if (s.tp != 1 && s.tp != 2 && s.tp != 4 && s.tp != 8)
    throw std::invalid_argument("tensor parallel degree must be 1, 2, 4 or 8");
  if (s.heads % s.tp || s.kv_heads % s.tp || s.inter % s.tp || s.vocab % s.tp)
    throw std::invalid_argument("heads, KV heads, intermediate size and vocabulary must divide by the tp degree");
  s.heads /= s.tp;
  s.kv_heads /= s.tp;
  s.inter /= s.tp;
  s.head_rows = s.vocab / s.tp;
  if (s.tp > 1 && s.head_dim != 128) throw std::invalid_argument("tensor-parallel plans are built for head_dim 128");
  if ((s.experts || s.qk_norm) && s.head_dim != 128)
    throw std::invalid_argument("mixture-of-experts / QK-norm plans are built for head_dim 128");
  if (s.tp > 1 && s.hidden % 2) throw std::invalid_argument("hidden size must be even for the all-reduce packets");
  if (s.tp > 1 && s.vocab > (1 << 20)) throw std::invalid_argument("the argmax exchange packet holds 20 index bits");
  if (s.experts && s.tp != 1) throw std::invalid_argument("tensor parallel mixture of experts is not built");
  s.batch_lo = int(plan.integer("batch_lo", 1));
  s.batch_hi = int(plan.integer("batch_hi", s.batch_lo));
  if (s.experts && s.batch_hi > kMaxBatch) throw std::invalid_argument("mixture-of-experts plans are built for batch 1..8");
  s.capacity = int(plan.integer("capacity", 0));
  s.dense_batch = s.batch_hi > kMaxBatch || s.prefill;
  if (s.prefill) {
    // the batch interval counts sequences; the kernel's rows are (sequence, position) pairs, 64 per step
    s.prefill_seq = int(plan.integer("seq", 0));
    if (s.batch_lo < 1 || s.batch_hi < s.batch_lo || s.batch_hi > kDenseMaxBatch)
      throw std::invalid_argument("a prefill plan covers 1..64 sequences");
    if (s.prefill_seq < 1 || s.prefill_seq >= s.capacity) throw std::invalid_argument("seq must lie in [1, capacity)");
  }
  if (s.dense_batch) {
    if (!s.prefill &&
        (s.batch_lo <= kMaxBatch || s.batch_hi > kDenseMaxBatch || s.batch_lo % 16 || s.batch_hi % 16 || s.batch_hi < s.batch_lo))
      throw std::invalid_argument("a dense-batch plan covers batch sizes 16, 32, 48, 64 (interval bounds multiples of 16)");
    if (s.head_dim != 128 || s.tp != 1 || s.experts || s.qk_norm || s.hidden > 8192)
      throw std::invalid_argument("dense-batch plans are built for unsharded dense models with head_dim 128 and hidden <= 8192");
  } else if (s.batch_lo < 1 || s.batch_hi < s.batch_lo) {
    throw std::invalid_argument("batch interval must lie in [1, 8] (or in [16, 64] in steps of 16 for a dense-batch plan)");
  }
  if (s.capacity < 2 || s.capacity % kKvBlock) throw std::invalid_argument("capacity must be a positive multiple of 16");
  const Json empty;
  const Json& kv = plan.has("kv") ? plan.at("kv") : empty;
  // "chunk_rows": rows of the batch may be consecutive positions of one sequence (their block-table rows name
  // the same pool blocks): every row's key and value are appended before any row attends (chunked prefill)
  s.chunk_rows = plan.flag("chunk_rows", false) || s.prefill;
  if (s.chunk_rows && !s.dense_batch) throw std::invalid_argument("chunk_rows needs a dense-batch plan (batch 16..64)");
  const std::string layout = kv.str("layout", "contiguous");
  if (layout != "contiguous" && layout != "paged") throw std::invalid_argument("kv.layout must be contiguous or paged");
  s.paged = layout == "paged";
  s.max_blocks = s.capacity / kKvBlock;
  if (s.paged) {
    s.num_blocks = int(kv.integer("num_blocks", 0));
    if (s.num_blocks < 1) throw std::invalid_argument("kv.num_blocks must be positive for a paged plan");
  }
  s.grid = int(plan.integer("grid", 0));
  s.slots = int(plan.integer("slots", 0));
  s.attn_min_slots = int(plan.integer("attn_min_slots", s.attn_min_slots));
  if (s.attn_min_slots < 1 || s.attn_min_slots > 64) throw std::invalid_argument("attn_min_slots must lie in [1, 64]");
  s.write_logits = plan.flag("write_logits", true);
  const Json& geometry = plan.has("geometry") ? plan.at("geometry") : empty;
  // "weights": "e4m3": every GEMV matrix as e4m3 bytes with one fp32 scale per output row (the scale
  // is applied to the fp32 sum before the stage's rounding sites); pages are 8 rows x 4096 columns
  const std::string weights = plan.str("weights", "bf16");
  if (weights != "bf16" && weights != "e4m3") throw std::invalid_argument("weights must be bf16 or e4m3");
  s.fp8 = weights == "e4m3";
  if (s.fp8 && (s.dense_batch || s.experts || s.head_dim != 128))
    throw std::invalid_argument("e4m3 weights are built for dense models with head_dim 128 at batch 1..8");
  const int elem = s.fp8 ? 1 : 2;
  s.geo[kQkv] = MakeGeo("qkv", s.qkv_rows(), s.hidden, geometry, elem);
  s.geo[kOProj] = MakeGeo("o", s.hidden, s.heads * s.head_dim, geometry, elem);
  s.geo[kGateUp] = MakeGeo("gate_up", 2 * s.inter, s.hidden, geometry, elem);
  s.geo[kDown] = MakeGeo("down", s.hidden, s.inter, geometry, elem);
  s.geo[kHead] = MakeGeo("lm_head", s.head_rows, s.hidden, geometry, elem);
  // A wide batch times a long down reduction does not fit in shared memory beside the ring
  // (8 rows x 14336 columns are 229 KB): the reduction is then cut into parts of whole pages
  // whose rows take about 80 KB, one stage per part, fp32 running sums in global memory.
  if (s.dense_batch) {
    const int sms = 148;   // the task count aims at two per SM of a B200; any grid runs it
    s.dgeo[kQkv] = MakeDenseGeo("qkv", s.qkv_rows(), s.hidden, sms);
    s.dgeo[kOProj] = MakeDenseGeo("o", s.hidden, s.heads * s.head_dim, sms);
    s.dgeo[kGateUp] = MakeDenseGeo("gate_up", 2 * s.inter, s.hidden, sms);
    s.dgeo[kDown] = MakeDenseGeo("down", s.hidden, s.inter, sms);
    s.dgeo[kHead] = MakeDenseGeo("lm_head", s.head_rows, s.hidden, sms);
    for (int g : {kQkv, kOProj, kGateUp, kDown, kHead}) s.geo[g] = StreamGeo(s.dgeo[g]);
  } else if (!s.experts) {
    const GemvGeo& down = s.geo[kDown];
    const int budget_columns = 81920 / (2 * s.batch_hi) - 8;   // activation rows are 2-byte elements whatever the weights are
    const int part_pages = std::max(1, std::min(down.pages_per_task, budget_columns / down.tile_k));
    s.down_splits = (down.pages_per_task + part_pages - 1) / part_pages;
    if (s.down_splits > kMaxDownSplits) throw std::invalid_argument("down projection would need more than 8 parts");
    for (int i = 0; i < s.down_splits; ++i) {
      GemvGeo part = down;
      part.page0 = i * part_pages;
      part.pages_per_task = std::min(part_pages, down.pages_per_task - part.page0);
      part.k = part.pages_per_task * down.tile_k;
      part.src_off = part.page0 * down.tile_k;
      part.k_src = std::min(part.k, down.k_src - part.src_off);
      const bool last = i + 1 == s.down_splits;
      part.last_page_bytes = last ? down.last_page_bytes : down.page_bytes;
      const int task_bytes = (part.pages_per_task - 1) * down.page_bytes + part.last_page_bytes;
      part.claim_chunk = std::max(1, std::min(8, (65536 + task_bytes - 1) / task_bytes));
      s.down_part[i] = part;
    }
  }
  if (s.experts) {
    s.geo[kRouter] = MakeGeo("router", s.experts, s.hidden, geometry);
    if (s.geo[kDown].pages_per_task != 1)
      throw std::invalid_argument("expert intermediate size must fit one 2048-column page");
  }

  auto add = [&](std::string name, uint32_t role, uint32_t dtype, uint64_t constant, uint64_t per_batch,
                 std::string recipe) {
    BufferSpec b;
    b.name = std::move(name);
    b.role = role;
    b.dtype = dtype;
    b.elements_constant = constant;
    b.elements_per_batch = per_batch;
    b.pack_json = std::move(recipe);
    s.buffers.push_back(std::move(b));
    return int(s.buffers.size()) - 1;
  };
  const uint64_t H = s.hidden, D = s.head_dim, V = s.vocab, I = s.inter;
  s.tokens = add("serving.tokens", 1, 2, 0, s.capacity, "");
  s.rope_cos = add("serving.rope_cos", 1, 0, uint64_t(s.capacity) * D, 0, "");
  s.rope_sin = add("serving.rope_sin", 1, 0, uint64_t(s.capacity) * D, 0, "");
  if (s.paged) {
    s.block_table = add("serving.block_table", 1, 2, 0, s.max_blocks, "");
    s.context_base = add("serving.context_base", 1, 2, 0, 1, "");
  }
  s.embed = add("model.embed_tokens.weight", 1, 0, V * H, 0, Alias("model.embed_tokens.weight"));
  // activation buffers hold one row per row of the kernel's batch: per sequence in a decode plan, a fixed
  // kDenseMaxBatch rows in a prefill plan (whose batch counts sequences)
  auto act = [&](const char* name, uint32_t dtype, uint64_t per_row) {
    return s.prefill ? add(name, 0, dtype, uint64_t(kDenseMaxBatch) * per_row, 0, "") : add(name, 0, dtype, 0, per_row, "");
  };
  // a prefill plan's GEMM weights are packed as 128 x 128 pages, a small-batch decode plan's as 8 x 2048: the
  // names differ so that a driver can hold both plans' buffers in one table (python/tilemega/serving/engine.py:49-57)
  const std::string wp = s.prefill ? "prefill." : "";
  s.hidden_buf = act("serving.hidden", 0, H);
  if (s.dense_batch) s.normed_buf = act("serving.normed", 0, H);   // RMSNorm output read by the GEMM stages
  // weight pages: 8 rows x 2048 columns for the GEMV path, 128 x 128 (a tcgen05 operand tile) for dense-batch plans
  const int page_n = s.dense_batch ? kDenseTileN : kTileN;
  auto page_k = [&](int stage) { return s.dense_batch ? kDenseTileK : s.geo[stage].tile_k; };
  const int swiglu_unit = s.dense_batch ? 16 : 4;   // gate rows followed by as many up rows
  // e4m3 plans: the matrix is quantised row by row ("e4m3_pairs": its bytes seen as 2-byte units, so
  // that tile_pages and its 128-byte swizzle apply unchanged: a page of 8 x 2048 units is 8 x 4096
  // e4m3 columns) and the row scales travel as an fp32 buffer of their own ("e4m3_scale")
  const uint32_t weight_dtype = s.fp8 ? 4u : 0u;
  auto weight_pages = [&](const std::string& source, int stage) {
    if (!s.fp8) return Pages(source, page_k(stage), page_n);
    return Pages("{\"kind\":\"e4m3_pairs\",\"source\":" + source + "}", 2048, kTileN);
  };
  auto scale_of = [&](const std::string& name, const std::string& source, int rows) {
    return s.fp8 ? add(name, 1, 1, uint64_t(rows), 0, "{\"kind\":\"e4m3_scale\",\"source\":" + source + "}") : -1;
  };
  s.qkv_buf = act("serving.qkv", 0, uint64_t(s.qkv_rows()));
  s.attn_buf = act("serving.attention", 0, uint64_t(s.heads) * D);
  // with experts: one row per chosen expert of the token being served (tokens take turns)
  s.mlp_buf = act("serving.mlp", 0, s.experts ? I * uint64_t(s.topk) : I);
  if (s.experts) {
    s.router_buf = add("serving.router_logits", 0, 0, 0, uint64_t(s.experts), "");
    // the experts chosen by the last step and their weights, [layers][batch][topk]
    s.route_idx_buf = add("serving.route_index", 0, 2, 0, uint64_t(s.layers) * s.topk, "");
    s.route_weight_buf = add("serving.route_weight", 0, 1, 0, uint64_t(s.layers) * s.topk, "");
  }
  s.logits_buf = act("serving.logits", 1, uint64_t(s.head_rows));  // fp32 accumulators of this rank's head rows
  for (int l = 0; l < s.layers; ++l) {
    const std::string p = "l" + std::to_string(l) + ".";
    const std::string m = "model.layers." + std::to_string(l) + ".";
    LayerBuffers lb{};
    lb.norm1 = add(p + "norm1.weight", 1, 0, H, 0, Alias(m + "input_layernorm.weight"));
    const std::string qkv_source =
        "{\"kind\":\"qkv_group_interleave\",\"sources\":" +
        Sources({m + "self_attn.q_proj.weight", m + "self_attn.k_proj.weight", m + "self_attn.v_proj.weight"}) +
        ",\"hkv\":" + std::to_string(s.kv_heads) + ",\"qperkv\":" + std::to_string(s.heads / s.kv_heads) +
        ",\"head_dim\":" + std::to_string(s.head_dim) + Shard(0, s.tp) + "}";
    lb.qkv = add(wp + p + "qkv.weight", 1, weight_dtype, uint64_t(s.geo[kQkv].n) * s.geo[kQkv].k, 0, weight_pages(qkv_source, kQkv));
    lb.qkv_scale = scale_of(p + "qkv.scale", qkv_source, s.geo[kQkv].n);
    if (s.paged) {
      const uint64_t pool = uint64_t(s.num_blocks) * s.kv_heads * kKvBlock * D;
      lb.k = add("kv_pool.k." + std::to_string(l), 1, 0, pool, 0, "");
      lb.v = add("kv_pool.v." + std::to_string(l), 1, 0, pool, 0, "");
    } else {
      const uint64_t cache = uint64_t(s.kv_heads) * s.capacity * D;
      lb.k = add("kv_cache.k." + std::to_string(l), 1, 0, 0, cache, "");
      lb.v = add("kv_cache.v." + std::to_string(l), 1, 0, 0, cache, "");
    }
    const std::string o_source = Alias(m + "self_attn.o_proj.weight", Shard(1, s.tp));
    lb.o = add(wp + p + "o.weight", 1, weight_dtype, uint64_t(s.geo[kOProj].n) * s.geo[kOProj].k, 0, weight_pages(o_source, kOProj));
    lb.o_scale = scale_of(p + "o.scale", o_source, s.geo[kOProj].n);
    lb.norm2 = add(p + "norm2.weight", 1, 0, H, 0, Alias(m + "post_attention_layernorm.weight"));
    if (s.qk_norm) {
      lb.q_norm = add(p + "q_norm.weight", 1, 0, D, 0, Alias(m + "self_attn.q_norm.weight"));
      lb.k_norm = add(p + "k_norm.weight", 1, 0, D, 0, Alias(m + "self_attn.k_norm.weight"));
    }
    if (s.experts) {
      // the reference's expert_stack recipe (python/tilemega/moe/weights.py:15-47): every
      // expert packed by itself, the packed experts one after the other
      auto stack = [&](const char* part) {
        return "{\"kind\":\"expert_stack\",\"prefix\":" + Json::Quote(m + "mlp.experts.") + ",\"part\":\"" + part +
               "\",\"experts\":" + std::to_string(s.experts) + ",\"hidden\":" + std::to_string(s.hidden) +
               ",\"intermediate\":" + std::to_string(s.inter) + ",\"u\":4}";
      };
      lb.router = add(p + "router.weight", 1, 0, uint64_t(s.geo[kRouter].n) * s.geo[kRouter].k, 0,
                      Pages(Alias(m + "mlp.gate.weight"), s.geo[kRouter].tile_k));
      lb.gate_up = add(p + "gate_up.weight", 1, 0, uint64_t(s.experts) * s.geo[kGateUp].n * s.geo[kGateUp].k, 0,
                       Pages(stack("gate_up"), s.geo[kGateUp].tile_k));
      lb.down = add(p + "down.weight", 1, 0, uint64_t(s.experts) * s.geo[kDown].n * s.geo[kDown].k, 0,
                    Pages(stack("down"), s.geo[kDown].tile_k));
      s.layer.push_back(lb);
      continue;
    }
    const std::string gate_up_source = "{\"kind\":\"gate_up_interleave\",\"sources\":" +
                                       Sources({m + "mlp.gate_proj.weight", m + "mlp.up_proj.weight"}) +
                                       ",\"u\":" + std::to_string(swiglu_unit) + Shard(0, s.tp) + "}";
    lb.gate_up = add(wp + p + "gate_up.weight", 1, weight_dtype, uint64_t(s.geo[kGateUp].n) * s.geo[kGateUp].k, 0,
                     weight_pages(gate_up_source, kGateUp));
    lb.gate_up_scale = scale_of(p + "gate_up.scale", gate_up_source, s.geo[kGateUp].n);
    const std::string down_source = Alias(m + "mlp.down_proj.weight", Shard(1, s.tp));
    lb.down = add(wp + p + "down.weight", 1, weight_dtype, uint64_t(s.geo[kDown].n) * s.geo[kDown].k, 0, weight_pages(down_source, kDown));
    lb.down_scale = scale_of(p + "down.scale", down_source, s.geo[kDown].n);
    s.layer.push_back(lb);
  }
  s.final_norm = add("model.norm.weight", 1, 0, H, 0, Alias("model.norm.weight"));
  const std::string head_source = Alias("lm_head.weight", Shard(0, s.tp));
  s.lm_head = add(wp + "lm_head.weight", 1, weight_dtype, uint64_t(s.geo[kHead].n) * s.geo[kHead].k, 0, weight_pages(head_source, kHead));
  s.lm_head_scale = scale_of("lm_head.scale", head_source, s.geo[kHead].n);
  return s;
}

}  // namespace tmb
