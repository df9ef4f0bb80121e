// Host-only planning entry points of the C ABI: which op chains fold into the GEMM's epilogue (the matmul pattern
// of the reference's fusion engine), the shard plan of the row-sharded product, and the code generator's
// "generate_matmul" answer for a library of precompiled kernels. Nothing here touches a GPU.
#include <cctype>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/symplex_b200.h"
#include "host_api.h"

namespace sx {
namespace {

enum OpKind { OP_OTHER, OP_MATMUL, OP_ADD, OP_MUL, OP_ACT };

struct ParsedOp {
  OpKind kind;
  int act;  // SYMPLEX_ACT_* when kind == OP_ACT
  long long bytes;
  int rank;
  std::string dtype;  // canonical name
};

std::string lower(const char* s) {
  std::string r = s ? s : "";
  for (char& c : r) c = (char)tolower((unsigned char)c);
  return r;
}

// DType::size_bytes of the reference (rust-engine/src/fusion_engine.rs:73-82); unknown names are fp32, as in
// discover_fusions' dtype match (rust-engine/src/lib.rs:378-385).
long long dtype_bytes(const char* name) {
  const std::string d = lower(name);
  if (d == "fp16" || d == "bf16") return 2;
  if (d == "fp8" || d == "int8" || d == "int4") return 1;
  return 4;
}

ParsedOp parse(const symplex_fusion_op& op) {
  ParsedOp p{OP_OTHER, SYMPLEX_ACT_NONE, 0, op.shape ? op.rank : 0, lower(op.dtype)};
  if (p.dtype != "fp16" && p.dtype != "bf16" && p.dtype != "fp8" && p.dtype != "int8" && p.dtype != "int4") p.dtype = "fp32";
  const std::string n = lower(op.op);
  if (n == "matmul" || n == "batch_matmul") p.kind = OP_MATMUL;
  else if (n == "add") p.kind = OP_ADD;
  else if (n == "mul") p.kind = OP_MUL;
  else if (n == "relu") { p.kind = OP_ACT; p.act = SYMPLEX_ACT_RELU; }
  else if (n == "gelu") { p.kind = OP_ACT; p.act = SYMPLEX_ACT_GELU; }
  else if (n == "sigmoid") { p.kind = OP_ACT; p.act = SYMPLEX_ACT_SIGMOID; }
  else if (n == "tanh") { p.kind = OP_ACT; p.act = SYMPLEX_ACT_TANH; }
  else if (n == "silu") { p.kind = OP_ACT; p.act = SYMPLEX_ACT_SILU; }
  long long elems = 1;  // memory_bytes = product(shape) * size_bytes (rust-engine/src/lib.rs:386)
  for (int i = 0; i < op.rank && op.shape != nullptr; ++i) elems *= op.shape[i];
  p.bytes = elems * dtype_bytes(op.dtype);
  return p;
}

// matches_matmul_bias_activation (rust-engine/src/fusion_engine.rs:1587-1623) on a window of 2..4 ops.
bool matches(const ParsedOp* o, size_t n) {
  if (n < 2 || n > 4 || o[0].kind != OP_MATMUL) return false;
  if (n == 2) return o[1].kind == OP_ADD || o[1].kind == OP_ACT;
  if (n == 3) return (o[1].kind == OP_ADD && o[2].kind == OP_ACT) || o[1].kind == OP_ACT;
  return o[1].kind == OP_MUL && o[2].kind == OP_ADD && o[3].kind == OP_ACT;
}

struct Epi {
  int act = SYMPLEX_ACT_NONE;
  bool bias = false, scale = false;
  size_t consumed = 0;
};

// The longest prefix [matmul, (mul,) (add,) (activation)] the kernel's epilogue act(alpha * acc + bias) executes.
bool compile(const ParsedOp* o, size_t n, Epi* e) {
  if (n == 0 || o[0].kind != OP_MATMUL) return false;
  size_t i = 1;
  if (i + 1 < n && o[i].kind == OP_MUL && o[i + 1].kind == OP_ADD) { e->scale = true; ++i; }
  if (i < n && o[i].kind == OP_ADD) { e->bias = true; ++i; }
  if (i < n && o[i].kind == OP_ACT) { e->act = o[i].act; ++i; }
  e->consumed = i;
  return true;
}

}  // namespace
}  // namespace sx

using namespace sx;

extern "C" {

int64_t symplex_b200_discover_fusions(const symplex_fusion_op* ops, size_t n_ops, char* json_out, size_t cap) {
  if ((ops == nullptr && n_ops != 0) || (json_out == nullptr && cap != 0))
    return set_last_error(SX_ERR_INVALID, "discover_fusions: null argument");
  std::vector<ParsedOp> po(n_ops);
  for (size_t i = 0; i < n_ops; ++i) po[i] = parse(ops[i]);
  struct Boundary { size_t first, count; long long savings; double confidence; };
  std::vector<Boundary> found;
  long long total = 0;
  for (size_t i = 0; i < n_ops;) {
    Epi e;
    if (compile(po.data() + i, n_ops - i, &e) && e.consumed >= 2 && matches(po.data() + i, e.consumed)) {
      // estimate_memory_savings(MatMulBiasReLU) (rust-engine/src/fusion_engine.rs:1209-1225): the matmul output and
      // the second op's output each cost one write and one read when the chain is not fused.
      const long long savings = 2 * po[i].bytes + 2 * po[i + 1].bytes;
      // compute_confidence (rust-engine/src/fusion_engine.rs:1882-1965): base 0.9 for this pattern, + 0.1 if all
      // ranked outputs have one rank, + 0.05 for one dtype, + 0.05 if an intermediate exceeds 1 MiB, + 0.05 when no
      // op is in place (discover_fusions never marks one so), clamped to [0, 1].
      double conf = 0.9;
      bool same_rank = true, same_dtype = true, large = false, any_rank = false;
      int rank0 = 0;
      for (size_t k = 0; k < e.consumed; ++k) {
        const ParsedOp& o = po[i + k];
        if (o.rank > 0) {
          if (!any_rank) { rank0 = o.rank; any_rank = true; }
          else if (o.rank != rank0) same_rank = false;
        }
        if (o.dtype != po[i].dtype) same_dtype = false;
        if (k + 1 < e.consumed && o.bytes > 1024 * 1024) large = true;
      }
      if (any_rank && same_rank) conf += 0.1;
      if (same_dtype) conf += 0.05;
      if (large) conf += 0.05;
      conf += 0.05;
      if (conf > 1.0) conf = 1.0;
      found.push_back({i, e.consumed, savings, conf});
      total += savings;
      i += e.consumed;
    } else {
      ++i;
    }
  }
  // Schema and number formats of rust-engine/src/lib.rs:398-412 ({:.3}, {:.2}, Rust's Debug print of Vec<usize>).
  // total_estimated_speedup: product over the boundaries of compute factor 1.1 x (1 + MB / (MB + 10)) x confidence
  // (FusionBoundary::estimated_speedup, rust-engine/src/fusion_engine.rs:784-802; FusionDecision::new, :859-873).
  double speedup = 1.0;
  for (size_t b = 0; b < found.size(); ++b) {
    const double mb = (double)found[b].savings / (1024.0 * 1024.0);
    speedup *= 1.1 * (mb > 0.0 ? 1.0 + mb / (mb + 10.0) : 1.0) * found[b].confidence;
  }
  std::string js = "{\n";
  char buf[256];
  snprintf(buf, sizeof(buf), "  \"total_estimated_speedup\": %.3f,\n", speedup);
  js += buf;
  snprintf(buf, sizeof(buf), "  \"total_hbm_traffic_reduction\": %lld,\n", total);
  js += buf;
  js += std::string("  \"requires_polyhedral_validation\": ") + (found.empty() ? "false" : "true") + ",\n";
  js += "  \"boundaries\": [\n";
  for (size_t b = 0; b < found.size(); ++b) {
    js += "    {\"op_indices\": [";
    for (size_t k = 0; k < found[b].count; ++k) {
      snprintf(buf, sizeof(buf), "%s%zu", k ? ", " : "", found[b].first + k);
      js += buf;
    }
    snprintf(buf, sizeof(buf),
             "], \"pattern\": \"MatMulBiasReLU\", \"memory_traffic_savings_bytes\": %lld, "
             "\"compute_savings_factor\": %.2f, \"confidence\": %.2f}",
             found[b].savings, 1.1, found[b].confidence);
    js += buf;
    if (b + 1 < found.size()) js += ",";
    js += "\n";
  }
  js += "  ]\n}\n";
  if (js.size() + 1 > cap) return -(int64_t)(js.size() + 1);
  memcpy(json_out, js.c_str(), js.size() + 1);
  return (int64_t)js.size();
}

int symplex_b200_compile_epilogue(const symplex_fusion_op* ops, size_t n_ops, size_t first, symplex_gemm_desc* d,
                                  int32_t* consumed, int32_t* has_bias, int32_t* has_scale) {
  if (ops == nullptr || d == nullptr) return set_last_error(SX_ERR_INVALID, "compile_epilogue: null argument");
  if (first >= n_ops) return set_last_error(SX_ERR_INVALID, "compile_epilogue: first op out of range");
  std::vector<ParsedOp> po(n_ops - first);
  for (size_t i = first; i < n_ops; ++i) po[i - first] = parse(ops[i]);
  Epi e;
  if (!compile(po.data(), po.size(), &e))
    return set_last_error(SX_ERR_INVALID, "compile_epilogue: the chain does not start with a matmul");
  d->activation = e.act;
  if (consumed) *consumed = (int32_t)e.consumed;
  if (has_bias) *has_bias = e.bias ? 1 : 0;
  if (has_scale) *has_scale = e.scale ? 1 : 0;
  return SX_OK;
}

int symplex_b200_analyze_matmul(int64_t M, int64_t N, int64_t K, int32_t world, int32_t bytes_per_element,
                                symplex_shard_plan* out) {
  if (out == nullptr) return set_last_error(SX_ERR_INVALID, "analyze_matmul: null output");
  memset(out, 0, sizeof(*out));
  if (world < 1 || M < 0 || N < 0 || K < 0 || bytes_per_element < 1)
    return set_last_error(SX_ERR_INVALID, "analyze_matmul: bad argument");
  if (M % world != 0) return set_last_error(SX_ERR_INVALID, "analyze_matmul: M rows do not split evenly over the devices");
  const int64_t m_loc = M / world, b = bytes_per_element;
  out->a = {1, 0, {M, K}, {m_loc, K}};   // SHARD_DIM_0
  out->b = {0, -1, {K, N}, {K, N}};      // REPLICATE
  out->c = {1, 0, {M, N}, {m_loc, N}};   // SHARD_DIM_0, then all-gathered
  out->world = world;
  if (world > 1) {
    out->n_all_gather_ops = 1;
    out->total_communication_bytes = (int64_t)world * (world - 1) * m_loc * N * b;
  }
  out->peak_memory_per_device = (m_loc * K + K * N + M * N) * b;
  return SX_OK;
}

void poly_get_micro_kernel_config(uint8_t target, size_t element_bytes, size_t* out_tile_m, size_t* out_tile_n,
                                  size_t* out_tile_k, size_t* out_acc_regs, size_t* out_prefetch_dist) {
  symplex_b200_micro_kernel_config(target, element_bytes, out_tile_m, out_tile_n, out_tile_k, out_acc_regs,
                                   out_prefetch_dist);
}

int symplex_b200_generate_matmul(int64_t M, int64_t N, int64_t K, int32_t element_bytes, int64_t tile_m, int64_t tile_n,
                                 int64_t tile_k, symplex_generated_kernel* out) {
  (void)tile_m;
  (void)tile_k;
  if (out == nullptr) return set_last_error(SX_ERR_INVALID, "generate_matmul: null output");
  memset(out, 0, sizeof(*out));
  if (element_bytes != 2 && element_bytes != 4) {
    snprintf(out->error_message, sizeof(out->error_message), "element size %d not on this path (2 = bf16, 4 = fp32)",
             element_bytes);
    return set_last_error(SX_ERR_INVALID, out->error_message);
  }
  symplex_gemm_desc d;
  const int32_t dt = element_bytes == 2 ? SYMPLEX_DT_BF16 : SYMPLEX_DT_F32;
  symplex_b200_gemm_desc_init(&d, M, N, K, dt, dt);
  if (tile_n == 64 || tile_n == 128 || tile_n == 256) d.tile_n = (int32_t)tile_n;  // other hints are repaired to auto
  symplex_gemm_plan plan;
  const int rc = symplex_b200_gemm_plan(&d, 0, &plan);
  if (rc != SX_OK) {
    strncpy(out->error_message, plan.error, sizeof(out->error_message) - 1);
    return rc;
  }
  strncpy(out->kernel_name, plan.kernel_name, sizeof(out->kernel_name) - 1);
  out->shared_mem_bytes = plan.shared_mem_bytes;
  const int64_t threads = plan.block_dims[0] > 0 ? plan.block_dims[0] : 1;
  int64_t regs = 65536 / threads / 8 * 8;
  out->register_count = regs > 255 ? 255 : regs;
  for (int i = 0; i < 3; ++i) {
    out->grid_dims[i] = plan.grid_dims[i];
    out->block_dims[i] = plan.block_dims[i];
  }
  out->valid = 1;
  return SX_OK;
}

}  // extern "C"
