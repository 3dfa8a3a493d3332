// Plan compiler and executor.
//
// A tensor plan (the reference's GpuExecutionPlan wire format, flattened to bg_plan_step) is
// compiled once per distinct plan into a list of kernel launches and cached by content hash:
//   1. FUSED_ELEMENTWISE / ATTENTION_FORWARD steps are expanded into primitive nodes;
//   2. LOAD / RESHAPE / PERMUTE / BROADCAST_TO become strided views (no data movement);
//   3. elementwise nodes of equal shape and equal dependency depth are merged into fusion
//      groups (the reference's own groups are single-consumer chains of six opcodes,
//      packages/browsergrad-jit/src/python/_fusion.py:141-181; here CMP, WHERE, CAST, constants,
//      broadcast operands and multi-consumer values fuse too);
//   4. a REDUCE / FUSED_SOFTMAX / LAYER_NORM over trailing axes becomes the on-chip tail of the
//      group that produces its input;
//   5. each group is lowered to an EwProgram (register program) for the generic kernel;
//   6. MATMUL, INDEX, CROSS_ENTROPY lower to their own kernels;
//   7. units are scheduled topologically, intermediates are allocated stream-ordered at first
//      use and freed after their last reader.
#include "runtime.h"

#include <string.h>

#include <algorithm>
#include <set>
#include <sstream>

namespace bg {

struct View {
  int slot = -1;        // storage slot, -1 for constants
  int64_t off = 0;      // element offset into the slot
  int rank = 0;
  int64_t shape[kMaxRank] = {0};
  int64_t stride[kMaxRank] = {0};
  int dtype = BG_F32;
  bool is_const = false;
  double cf = 0;
  int64_t ci = 0;
  int64_t numel() const {
    int64_t n = 1;
    for (int i = 0; i < rank; ++i) n *= shape[i];
    return n;
  }
  bool contiguous() const {
    int64_t expect = 1;
    for (int d = rank - 1; d >= 0; --d) {
      if (shape[d] != 1 && stride[d] != expect) return false;
      expect *= shape[d];
    }
    return true;
  }
  void set_dense(const int64_t* shp, int r) {
    rank = r;
    int64_t s = 1;
    for (int d = r - 1; d >= 0; --d) {
      shape[d] = shp[d];
      stride[d] = s;
      s *= shp[d];
    }
  }
};

struct Node {
  int op = 0, dtype = BG_F32, rank = 0;
  int64_t shape[kMaxRank] = {0};
  std::vector<int> in;
  int64_t iarg[kMaxRank] = {0};
  double farg[2] = {0, 0};
  int step = -1;
  int64_t numel() const {
    int64_t n = 1;
    for (int i = 0; i < rank; ++i) n *= shape[i];
    return n;
  }
};

enum Kind { K_LEAF, K_CONST, K_ALIAS, K_VIEW, K_EW, K_ROW, K_OTHER, K_DEAD };

struct Slot {
  int64_t bytes = 0;
  bool external = false;
  int value_node = -1;   // for external slots: the BUFFER node
  int first_unit = -1, last_unit = -1;
};

struct Run {
  bg_context* ctx;
  std::vector<void*> ptr;
  std::vector<char> from_handle;   // slot is bound to a caller-owned handle (its contents outlive the run)
};

struct Unit {
  std::string name;
  std::vector<int> reads, writes;   // slots
  std::function<int(Run&)> fn;
  int launches = 1;
};

struct CompiledPlan {
  std::vector<Slot> slots;
  std::vector<Unit> units;
  std::vector<std::pair<int, int>> buffers;  // (step value_id, slot)
  std::vector<int64_t> buffer_bytes;
  int root_slot = -1;
  int root_dtype = BG_F32;
  int root_rank = 0;
  int64_t root_shape[kMaxRank] = {0};
  int64_t root_bytes = 0;
  // the bytes the plan was compiled from: a cache hit is a hit only when they are equal, not merely their hash
  std::vector<unsigned char> key_bytes;
  // The device status word: `uses_status` marks kernels that can refuse their data (an index outside its axis),
  // `uses_wait_status` kernels whose bounded device waits can give up (tensor-core pipelines).  A plan that returns
  // its root to the host synchronises anyway and examines the word before it hands anything back, so the refusal is
  // raised at the call, as the reference raises it.  A plan that keeps its root on the device does not wait: the word
  // is copied to the host behind the plan and examined by the next call that synchronises or starts another plan --
  // always before any byte computed from the refused data can reach the host.
  bool uses_status = false;
  bool uses_wait_status = false;
  int64_t plan_peak = 0;
  std::string trace;
};

namespace {

inline EwType cls_of(int dt) {
  if (dt == BG_F64) return T_F64;
  if (dtype_is_float(dt)) return T_F32;
  if (dt == BG_BOOL) return T_B;
  return T_I64;
}
inline bool narrow_dtype(int dt) {
  return dt == BG_F16 || dt == BG_BF16 || dt == BG_I8 || dt == BG_I16 || dt == BG_I32 || dt == BG_U8 || dt == BG_U16 ||
         dt == BG_U32;
}
// np.promote_types for the dtypes of the IR (bfloat16 treated like float16 against integers).
int promote(int a, int b) {
  if (a == b) return a;
  if (a == BG_BOOL) return b;
  if (b == BG_BOOL) return a;
  const bool fa = dtype_is_float(a), fb = dtype_is_float(b);
  if (fa && fb) {
    if (a == BG_F64 || b == BG_F64) return BG_F64;
    if (a == BG_F32 || b == BG_F32) return BG_F32;
    return (a == b) ? a : BG_F32;  // f16 with bf16
  }
  if (fa || fb) {
    int f = fa ? a : b, i = fa ? b : a;
    int ibits = dtype_size(i) * 8;
    if (f == BG_F64) return BG_F64;
    if (f == BG_F32) return ibits <= 16 ? BG_F32 : BG_F64;
    return ibits <= 8 ? f : (ibits <= 16 ? BG_F32 : BG_F64);
  }
  const bool sa = a >= BG_I8 && a <= BG_I64, sb = b >= BG_I8 && b <= BG_I64;
  const int ba = dtype_size(a), bb = dtype_size(b);
  if (sa == sb) return ba >= bb ? a : b;
  int s = sa ? a : b, u = sa ? b : a;
  int bs = dtype_size(s), bu = dtype_size(u);
  if (bs > bu) return s;
  if (bu == 8) return BG_F64;
  return bu == 1 ? BG_I16 : (bu == 2 ? BG_I32 : BG_I64);
}

bool is_ew_op(int op) {
  switch (op) {
    case BG_OP_CAST: case BG_OP_ADD: case BG_OP_MUL: case BG_OP_DIV: case BG_OP_NEG: case BG_OP_EXP: case BG_OP_LOG:
    case BG_OP_ABS: case BG_OP_SIGN: case BG_OP_SIN: case BG_OP_COS: case BG_OP_ISNAN: case BG_OP_CMP: case BG_OP_WHERE:
      return true;
  }
  return false;
}

uint64_t fnv1a(const void* data, size_t n, uint64_t h) {
  const unsigned char* p = reinterpret_cast<const unsigned char*>(data);
  for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 1099511628211ull; }
  return h;
}

struct CompileError {
  int code;
  std::string msg;
};

// What a tensor-core GEMM unit applies to its accumulator before storing; filled in when the
// elementwise group that consumes the product is folded into the GEMM.
struct TcEpilogue {
  int out_slot = -1;     // >= 0: store here (the folded group's output) instead of the MATMUL slot
  int out_dtype = BG_F32;
  int bias_slot = -1;
  int64_t bias_off = 0;
  int bias_dtype = BG_F32;
  int act = TC_ACT_NONE;
  int round_acc = 0;
  int wide = 0;
};

// A fusion group lowered to a program, with slot references to patch at run time.
struct ProgramSpec {
  EwProgram prog;
  int in_slot[kEwMaxInputs];
  int64_t in_off_bytes[kEwMaxInputs];
  int out_slot[kEwMaxOutputs];
  bool row = false;
  int static_pattern = -1;   // >= 0: run the specialised kernel for this expression
  int static_kind = 0;
  int static_arg = 0;
  std::string signature;
  // layer norm over a sum of terms (ln_static.cu): operand index per term, output index of the stored sum
  int ln_terms = 0;
  int ln_term[4] = {0, 0, 0, 0};
  int ln_rowvec[4] = {0, 0, 0, 0};
  int ln_sum_out = -1;
  int ln_planes_hi = -1, ln_planes_lo = -1;   // slots of the normalised rows stored as split-product operand planes
  int ln_out16 = -1, ln_out16_dtype = 0;      // slot of the normalised rows stored in the 16-bit type of the GEMMs that read them
};

class Compiler {
 public:
  Compiler(bg_context* ctx, const bg_plan* plan) : ctx_(ctx), plan_(plan) {}
  std::shared_ptr<CompiledPlan> compile();

 private:
  bg_context* ctx_;
  const bg_plan* plan_;
  std::vector<Node> nodes_;
  std::vector<int> step_node_;
  std::vector<Kind> kind_;
  std::vector<View> view_;
  std::vector<std::vector<int>> cons_;
  std::vector<int> depth_, group_, need_mat_, tail_of_group_, attached_;
  std::vector<char> force_break_;
  std::vector<char> leaflike_;
  std::map<int, View> copy_src_;   // RESHAPE nodes that need a dense copy: the strided source view
  bool has_f64_leaf_ = false;
  std::map<int, std::shared_ptr<TcEpilogue>> tc_epilogues_;   // MATMUL node -> epilogue fused into its kernel
  std::map<int, int> tc_unit_of_;
  struct EpiPlan {
    int final_node = -1;   // node whose value the GEMM stores
    int bias_node = -1;
    int act = TC_ACT_NONE;
    int round_acc = 0;
    int wide = 0;
    int group = -1;
  };
  struct AttnPlan {
    int q = -1, kt = -1, v = -1;      // operand nodes (kt: the [B,H,D,Sk] view fed to the first MATMUL)
    int q_src = -1, kt_src = -1, v_src = -1;   // fp32 node behind an absorbed fp32 -> 16-bit CAST of that operand, or -1
    int mask = -1, mask_is_bool = 0;
    int scale_node = -1;              // BUFFER-backed multiplier, or -1 with scale_const
    double scale_const = 1.0;
    int mode = 1, ab_dtype = BG_F32;
    // RESHAPE node whose dense copy of PERMUTE(result) the kernel writes directly (head merge), or -1
    int out_node = -1;
    int64_t out_stride[3] = {0, 0, 0};   // element strides of the result over batch / head / query row
  };
  std::set<int> copy_elided_;             // RESHAPE copies produced by the attention kernel itself
  std::map<int, AttnPlan> attn_plan_;     // final MATMUL node -> fused attention
  std::set<int> attn_absorbed_;           // nodes that only exist inside a fused attention
  bool match_attention(int n, AttnPlan& ap, std::vector<int>& interior);
  void plan_attention();
  void emit_attention(int n, int key);
  void emit_shape_op(int n, int key);
  void emit_scatter(int n, int key);
  std::map<int, EpiPlan> epi_plan_;       // MATMUL node -> folded epilogue
  // MATMUL node -> fp32 nodes behind absorbed fp32 -> 16-bit CASTs of its A / B operand (-1: operand used as is)
  std::map<int, std::pair<int, int>> gemm_cast_src_;
  int absorbable_cast(int node, int dtype16, int& cast_node, bool allow_f64 = false);
  void plan_gemm_casts();
  // Tensor-core GEMMs of one plan that read the same A and differ only in their leaf B / bias (the q / k / v
  // projections of one activation) run as one launch: every member prepares its operands in a unit of its own,
  // the last member launches all of them and is the producer of every member's result.
  struct GroupRun {
    TcGemm g[3]; void* tmp[3]; size_t tmp_bytes[3];
    // where each member's result goes: resolved by the launching member, when every result slot exists
    std::shared_ptr<TcEpilogue> epi[3];
    int sc_slot[3], c_dt[3];
  };
  struct GemmGroup {
    std::vector<int> members;       // MATMUL nodes in node order
    std::vector<int> punits;        // units of the members emitted so far
    std::vector<int> finals;        // result nodes of the members emitted so far
    std::vector<int> keep_slots;    // scratch the members wrote that the joint launch reads
    std::shared_ptr<GroupRun> run;
  };
  std::vector<GemmGroup> gemm_groups_;
  std::map<int, int> gemm_group_of_;
  void plan_gemm_groups();
  std::map<std::tuple<int, int64_t, int64_t, int>, std::pair<int, int>> conv_memo_;   // fp32 A operand -> (16-bit slot, converting unit)
  std::set<int> absorbed_groups_;
  int tc_mode(int n);                      // -1: SIMT; 0: 16-bit operands; 1: 3xTF32
  bool small_gemm(int n, int* splits, int64_t* partial_bytes);   // a 2-D fp32 MATMUL the split-K small kernel takes
  bool storage_readers(int f, std::vector<int>& readers);   // who reads f's storage; false if it must hold f as typed
  bool feeds_only_split_gemms(int f);      // every reader of f is the dense A operand of a bf16-plane split product
  void publish_planes(int f, int hi, int lo, int punit);
  bool feeds_only_convert16(int f, int* dtype16);   // every reader of f is the absorbed 16-bit CAST of a GEMM's A operand
  bool feeds_only_attention32(int f);      // every reader of the fp64 value f is a fused 3xTF32 attention
  bool narrow_store(int n);                // the fp64 result of tensor-core MATMUL n is stored as the fp32 values it holds
  std::set<int> narrow32_slots_;           // slots of fp64 nodes that hold fp32 data (read only by the attention kernels)
  std::string act_expr(int node, int x, int g, int depth);
  void plan_tc_epilogues(const std::map<int, std::vector<int>>& groups);
  std::shared_ptr<CompiledPlan> cp_;
  int root_ = -1;
  // scheduling
  struct PUnit {
    Unit u;
    int order_key;
    std::vector<int> dep_nodes;   // nodes whose storage must be ready
    std::vector<int> out_nodes;   // nodes this unit makes ready
    std::vector<int> dep_punits;  // units whose scratch output this unit reads (index into punits_)
  };
  // hi / lo planes of a 3xTF32 operand, produced once per plan for every tensor-core GEMM that reads the same
  // dense operand: (slot, byte offset, elements) -> (hi slot, lo slot, producing unit)
  struct SplitMemo { int hi, lo, punit; };
  std::map<std::tuple<int, int64_t, int64_t>, SplitMemo> split_memo_;
  std::vector<PUnit> punits_;
  std::vector<int> producer_;     // node -> punit index (-1: always ready)

  [[noreturn]] void err(int code, const std::string& m) { throw CompileError{code, m}; }
  int new_slot(int64_t bytes, bool external, int node) {
    Slot s;
    s.bytes = bytes;
    s.external = external;
    s.value_node = node;
    cp_->slots.push_back(s);
    return (int)cp_->slots.size() - 1;
  }
  int resolve(int n) const {  // through LOAD aliases
    while (kind_[n] == K_ALIAS) n = nodes_[n].in[0];
    return n;
  }
  int find(int g) {
    while (group_[g] != g) { group_[g] = group_[group_[g]]; g = group_[g]; }
    return g;
  }
  void expand();
  void simplify();
  std::vector<char> live_;
  void build_views();
  void analyse();
  bool try_lower();
  void own_slot(int n) {
    if (view_[n].slot < 0) err(BG_ERR_INVALID, "internal: computed value without a slot");
  }
  bool build_program(const std::vector<int>& members, int tail_node, ProgramSpec& ps, std::vector<int>& dep_nodes,
                     std::vector<int>& out_nodes, std::string& why);
  void add_unit(PUnit&& pu) { punits_.push_back(std::move(pu)); }
  void emit_group(const std::vector<int>& members, int tail_node, int key);
  void emit_row_standalone(int r, int key);
  void emit_matmul(int n, int key);
  void emit_index(int n, int key);
  void emit_ce(int n, int key);
  void emit_copy(int n, const View& sv, int src, int key);
  void emit_generic_reduce(int n, int key);
  void emit_generic_softmax(int n, int key);
  void emit_const_fill(int n, int key);
  bool row_geometry(int r, int64_t& rows, int64_t& cols, View& xin, bool& trailing);
  void schedule();
};

void Compiler::expand() {
  const int ns = plan_->n_steps;
  step_node_.assign(ns, -1);
  for (int s = 0; s < ns; ++s) {
    const bg_plan_step& st = plan_->steps[s];
    if (st.op < 0 || st.op >= BG_OP_COUNT) err(BG_ERR_UNSUPPORTED, "plan step " + std::to_string(s) + ": unknown opcode");
    if (st.rank < 0 || st.rank > BG_MAX_RANK) err(BG_ERR_INVALID, "plan step " + std::to_string(s) + ": bad rank");
    if (!dtype_size(st.dtype)) err(BG_ERR_INVALID, "plan step " + std::to_string(s) + ": unknown dtype");
    if (st.n_inputs < 0 || st.n_inputs > BG_MAX_STEP_INPUTS) err(BG_ERR_INVALID, "plan step " + std::to_string(s) + ": bad input count");
    std::vector<int> ins;
    for (int i = 0; i < st.n_inputs; ++i) {
      int id = st.input_ids[i];
      if (id < 0 || id >= s) err(BG_ERR_INVALID, "plan step " + std::to_string(s) + ": input " + std::to_string(id) + " does not precede it");
      ins.push_back(step_node_[id]);
    }
    auto base = [&](int op) {
      Node n;
      n.op = op;
      n.dtype = st.dtype;
      n.rank = st.rank;
      for (int d = 0; d < st.rank; ++d) {
        if (st.shape[d] < 0) err(BG_ERR_INVALID, "plan step " + std::to_string(s) + ": negative extent");
        n.shape[d] = st.shape[d];
      }
      memcpy(n.iarg, st.iarg, sizeof(n.iarg));
      n.farg[0] = st.farg[0];
      n.farg[1] = st.farg[1];
      n.step = s;
      return n;
    };
    if (st.op == BG_OP_FUSED_ELEMENTWISE) {
      if (st.ext_count < 1 || st.ext_offset < 0 || (int64_t)st.ext_offset + 3ll * st.ext_count > plan_->n_ext)
        err(BG_ERR_INVALID, "FUSED_ELEMENTWISE: op list out of range");
      std::vector<int> made;
      for (int k = 0; k < st.ext_count; ++k) {
        const int32_t* t = plan_->ext + st.ext_offset + 3 * k;
        int op = t[0];
        if (!(op == BG_OP_ADD || op == BG_OP_MUL || op == BG_OP_DIV || op == BG_OP_NEG || op == BG_OP_EXP || op == BG_OP_LOG))
          err(BG_ERR_UNSUPPORTED, std::string("FUSED_ELEMENTWISE: unsupported inner opcode ") + op_name(op));
        auto ref = [&](int32_t r) -> int {
          if (r < 0) {
            int e = -r - 1;
            if (e >= (int)ins.size()) err(BG_ERR_INVALID, "FUSED_ELEMENTWISE: external ref out of range");
            return ins[e];
          }
          if (r >= k) err(BG_ERR_INVALID, "FUSED_ELEMENTWISE: step ref does not precede its use");
          return made[r];
        };
        Node n = base(op);
        n.in.push_back(ref(t[1]));
        const bool binary = op == BG_OP_ADD || op == BG_OP_MUL || op == BG_OP_DIV;
        if (binary) {
          if (t[2] == BG_REF_NONE) err(BG_ERR_INVALID, "FUSED_ELEMENTWISE: binary op without rhs");
          n.in.push_back(ref(t[2]));
        }
        nodes_.push_back(n);
        made.push_back((int)nodes_.size() - 1);
      }
      step_node_[s] = made.back();
    } else if (st.op == BG_OP_ATTENTION_FORWARD) {
      if (ins.size() != 3 || st.rank != 4) err(BG_ERR_INVALID, "ATTENTION_FORWARD: three rank-4 inputs required");
      const Node& q = nodes_[ins[0]];
      const Node& k = nodes_[ins[1]];
      if (q.rank != 4 || k.rank != 4) err(BG_ERR_INVALID, "ATTENTION_FORWARD: rank-4 inputs required");
      Node kt = base(BG_OP_PERMUTE);
      kt.shape[2] = k.shape[3]; kt.shape[3] = k.shape[2];
      kt.shape[0] = k.shape[0]; kt.shape[1] = k.shape[1];
      kt.in = {ins[1]};
      kt.iarg[0] = 0; kt.iarg[1] = 1; kt.iarg[2] = 3; kt.iarg[3] = 2;
      nodes_.push_back(kt);
      int ikt = (int)nodes_.size() - 1;
      Node mm = base(BG_OP_MATMUL);
      mm.shape[3] = k.shape[2];
      mm.in = {ins[0], ikt};
      nodes_.push_back(mm);
      int imm = (int)nodes_.size() - 1;
      Node c = base(BG_OP_CONST);
      c.rank = 0;
      c.farg[0] = (double)(float)st.farg[0];
      nodes_.push_back(c);
      int ic = (int)nodes_.size() - 1;
      Node mu = base(BG_OP_MUL);
      mu.shape[3] = k.shape[2];
      mu.in = {imm, ic};
      nodes_.push_back(mu);
      int imu = (int)nodes_.size() - 1;
      Node sm = base(BG_OP_FUSED_SOFTMAX);
      sm.shape[3] = k.shape[2];
      sm.in = {imu};
      sm.iarg[0] = 3;
      nodes_.push_back(sm);
      int ism = (int)nodes_.size() - 1;
      Node pv = base(BG_OP_MATMUL);
      pv.in = {ism, ins[2]};
      nodes_.push_back(pv);
      step_node_[s] = (int)nodes_.size() - 1;
    } else {
      Node n = base(st.op);
      n.in = ins;
      nodes_.push_back(n);
      step_node_[s] = (int)nodes_.size() - 1;
    }
  }
  if (plan_->root_id < 0 || plan_->root_id >= ns) err(BG_ERR_INVALID, "plan root out of range");
  root_ = step_node_[plan_->root_id];
}

// Graph clean-up on the expanded node list:
//  * CAST of a CONST folds into a CONST of the target dtype (the AMP pass wraps Python-scalar
//    constants in CASTs, packages/browsergrad-jit/src/python/_amp.py:183-261);
//  * the six-node softmax template REDUCE(max) -> NEG -> ADD -> EXP -> REDUCE(sum) -> DIV is
//    rewritten to FUSED_SOFTMAX.  The reference's fuse pass does the same
//    (_fusion.py:273-351) but loses the rewrite when a node downstream is substituted too
//    (_fusion.py:383-388), so multi-layer graphs arrive with the primitive form;
//  * nodes the root does not depend on are dropped.
void Compiler::simplify() {
  const int nn = (int)nodes_.size();
  for (int i = 0; i < nn; ++i) {
    Node& n = nodes_[i];
    if (n.op == BG_OP_CAST && n.in.size() == 1 && nodes_[n.in[0]].op == BG_OP_CONST) {
      const Node& c = nodes_[n.in[0]];
      double cf = dtype_is_float(c.dtype) ? c.farg[0] : (double)c.iarg[0];
      int64_t ci = dtype_is_float(c.dtype) ? (int64_t)c.farg[0] : c.iarg[0];
      Node f = n;
      f.op = BG_OP_CONST;
      f.in.clear();
      if (n.dtype == BG_F32) f.farg[0] = (double)(float)cf;
      else if (n.dtype == BG_F64) f.farg[0] = cf;
      else if (dtype_is_float(n.dtype)) continue;  // f16 / bf16 rounding stays on the device
      else if (n.dtype == BG_BOOL) f.iarg[0] = dtype_is_float(c.dtype) ? (cf != 0.0) : (ci != 0);
      else if (n.dtype == BG_I64) f.iarg[0] = ci;
      else continue;
      n = f;
    }
  }
  // A CAST to the dtype its input already has changes nothing: it becomes a view (the AMP pass narrows the 16-bit
  // output of an attention block once more in front of the next Linear).
  for (int i = 0; i < nn; ++i) {
    Node& c = nodes_[i];
    if (c.op == BG_OP_CAST && c.in.size() == 1 && nodes_[c.in[0]].dtype == c.dtype && nodes_[c.in[0]].rank == c.rank) c.op = BG_OP_RESHAPE;
  }
  // CAST(PERMUTE(x)) -> PERMUTE(CAST(x)): the conversion then reads x densely and the permutation stays
  // a view (the AMP pass casts the transposed weight of every Linear, _amp.py:215-226).  Repeated until nothing
  // moves, so a cast sinks below a chain of permutations (the transposed keys of an attention block).
  for (bool moved = true; moved;) {
    moved = false;
    std::vector<int> n_uses(nn, 0);
    for (int i = 0; i < nn; ++i)
      for (int in : nodes_[i].in) n_uses[in]++;
    for (int i = 0; i < nn; ++i) {
      Node& c = nodes_[i];
      if (c.op != BG_OP_CAST || c.in.size() != 1) continue;
      const int pi = c.in[0];
      Node& pm = nodes_[pi];
      if (pm.op != BG_OP_PERMUTE || pm.in.size() != 1 || n_uses[pi] != 1 || pi == root_) continue;
      const Node& src = nodes_[pm.in[0]];
      Node cast = c;           // becomes node pi: CAST of the un-permuted source
      cast.in = pm.in;
      cast.rank = src.rank;
      for (int d = 0; d < src.rank; ++d) cast.shape[d] = src.shape[d];
      Node perm = pm;          // becomes node i: PERMUTE of the cast
      perm.in = {pi};
      perm.dtype = c.dtype;
      perm.step = c.step;
      nodes_[pi] = cast;
      nodes_[i] = perm;
      moved = true;
    }
  }
  // CAST to a 16-bit type of (views of) a CAST from that same type: both casts are exact inverses on these values
  // (the AMP pass widens an attention output to fp32 and narrows it again in front of the next Linear,
  // _amp.py:183-261).  Both become views, so the 16-bit tensor is read in place.
  {
    std::vector<int> n_uses(nn, 0);
    for (int i = 0; i < nn; ++i)
      for (int in : nodes_[i].in) n_uses[in]++;
    for (int i = 0; i < nn; ++i) {
      Node& c = nodes_[i];
      if (c.op != BG_OP_CAST || c.in.size() != 1 || (c.dtype != BG_F16 && c.dtype != BG_BF16)) continue;
      std::vector<int> chain;
      int v = c.in[0];
      while ((nodes_[v].op == BG_OP_PERMUTE || nodes_[v].op == BG_OP_RESHAPE) && nodes_[v].in.size() == 1 && n_uses[v] == 1 && v != root_) {
        chain.push_back(v);
        v = nodes_[v].in[0];
      }
      Node& w = nodes_[v];
      if (w.op != BG_OP_CAST || w.in.size() != 1 || n_uses[v] != 1 || v == root_) continue;
      if ((w.dtype != BG_F32 && w.dtype != BG_F64) || nodes_[w.in[0]].dtype != c.dtype) continue;
      const int rank_w = w.rank;
      w.op = BG_OP_RESHAPE;          // same shape: a view of its 16-bit input
      w.dtype = c.dtype;
      (void)rank_w;
      for (int u : chain) nodes_[u].dtype = c.dtype;
      c.op = BG_OP_RESHAPE;
    }
  }
  auto compute_live = [&]() {
    live_.assign(nn, 0);
    std::vector<int> stack{root_};
    while (!stack.empty()) {
      int x = stack.back();
      stack.pop_back();
      if (live_[x]) continue;
      live_[x] = 1;
      for (int in : nodes_[x].in) stack.push_back(in);
    }
  };
  compute_live();
  std::vector<int> uses(nn, 0);
  for (int i = 0; i < nn; ++i)
    if (live_[i])
      for (int in : nodes_[i].in) uses[in]++;
  auto single_axis = [&](const Node& r, int& axis) {
    uint64_t m = (uint64_t)r.iarg[1];
    if (m == 0 || (m & (m - 1))) return false;
    axis = 0;
    while (!((m >> axis) & 1)) ++axis;
    return true;
  };
  bool changed = false;
  for (int i = 0; i < nn; ++i) {
    Node& div = nodes_[i];
    if (!live_[i] || div.op != BG_OP_DIV || div.in.size() != 2) continue;
    const int ie = div.in[0], is = div.in[1];
    const Node& e = nodes_[ie];
    const Node& sum = nodes_[is];
    int ax_s, ax_m;
    if (e.op != BG_OP_EXP || sum.op != BG_OP_REDUCE || sum.iarg[0] != BG_RED_SUM || !sum.iarg[2]) continue;
    if (sum.in.size() != 1 || sum.in[0] != ie || uses[ie] != 2 || uses[is] != 1 || !single_axis(sum, ax_s)) continue;
    const int ia = e.in[0];
    const Node& add = nodes_[ia];
    if (add.op != BG_OP_ADD || add.in.size() != 2 || uses[ia] != 1) continue;
    int ix = add.in[0], ineg = add.in[1];
    if (nodes_[ineg].op != BG_OP_NEG) std::swap(ix, ineg);
    const Node& neg = nodes_[ineg];
    if (neg.op != BG_OP_NEG || uses[ineg] != 1) continue;
    const int im = neg.in[0];
    const Node& mx = nodes_[im];
    if (mx.op != BG_OP_REDUCE || mx.iarg[0] != BG_RED_MAX || !mx.iarg[2] || uses[im] != 1) continue;
    if (mx.in.size() != 1 || mx.in[0] != ix || !single_axis(mx, ax_m) || ax_m != ax_s) continue;
    if (nodes_[ix].rank != div.rank || nodes_[ix].dtype != div.dtype) continue;
    bool same = true;
    for (int d = 0; d < div.rank; ++d) same &= nodes_[ix].shape[d] == div.shape[d];
    if (!same) continue;
    div.op = BG_OP_FUSED_SOFTMAX;
    div.in = {ix};
    memset(div.iarg, 0, sizeof(div.iarg));
    div.iarg[0] = ax_s;
    changed = true;
    // uses of the absorbed nodes are stale now; recompute before the next match
    compute_live();
    std::fill(uses.begin(), uses.end(), 0);
    for (int k = 0; k < nn; ++k)
      if (live_[k])
        for (int in : nodes_[k].in) uses[in]++;
  }
  (void)changed;
}

void Compiler::build_views() {
  const int nn = (int)nodes_.size();
  kind_.assign(nn, K_OTHER);
  view_.assign(nn, View());
  leaflike_.assign(nn, 0);
  for (int i = 0; i < nn; ++i) {
    Node& n = nodes_[i];
    View& v = view_[i];
    v.dtype = n.dtype;
    if (!live_[i]) { kind_[i] = K_DEAD; continue; }
    auto need_inputs = [&](size_t k) {
      if (n.in.size() != k) err(BG_ERR_INVALID, std::string(op_name(n.op)) + ": expected " + std::to_string(k) + " inputs");
    };
    switch (n.op) {
      case BG_OP_BUFFER: {
        kind_[i] = K_LEAF;
        leaflike_[i] = 1;
        if (n.dtype == BG_F64) has_f64_leaf_ = true;
        v.set_dense(n.shape, n.rank);
        v.slot = new_slot(n.numel() * dtype_size(n.dtype), true, i);
        cp_->buffers.push_back({n.step, v.slot});
        cp_->buffer_bytes.push_back(n.numel() * dtype_size(n.dtype));
        break;
      }
      case BG_OP_CONST:
        kind_[i] = K_CONST;
        leaflike_[i] = 1;
        v.set_dense(n.shape, n.rank);
        v.is_const = true;
        if (dtype_is_float(n.dtype)) { v.cf = n.farg[0]; v.ci = (int64_t)n.farg[0]; }
        else { v.ci = n.iarg[0]; v.cf = (double)n.iarg[0]; }
        break;
      case BG_OP_LOAD:
        need_inputs(1);
        kind_[i] = K_ALIAS;
        leaflike_[i] = leaflike_[n.in[0]];
        v = view_[n.in[0]];
        break;
      case BG_OP_PERMUTE: {
        need_inputs(1);
        const int src = resolve(n.in[0]);
        if (nodes_[src].rank != n.rank) err(BG_ERR_INVALID, "PERMUTE: rank mismatch");
        std::set<int64_t> seen;
        for (int d = 0; d < n.rank; ++d) {
          int64_t a = n.iarg[d];
          if (a < 0 || a >= n.rank || !seen.insert(a).second) err(BG_ERR_INVALID, "PERMUTE: axes are not a permutation");
          if (nodes_[src].shape[a] != n.shape[d]) err(BG_ERR_INVALID, "PERMUTE: declared shape does not match permuted input");
        }
        kind_[i] = K_VIEW;
        break;
      }
      case BG_OP_BROADCAST_TO: case BG_OP_RESHAPE:
        need_inputs(1);
        kind_[i] = K_VIEW;
        break;
      case BG_OP_SLICE: {
        need_inputs(1);
        const Node& sn = nodes_[resolve(n.in[0])];
        if (sn.rank != n.rank) err(BG_ERR_INVALID, "SLICE: rank changes");
        for (int d = 0; d < n.rank; ++d) {
          const int64_t start = n.iarg[d] & (((int64_t)1 << 40) - 1), step = n.iarg[d] >> 40;
          if (step < 1 || n.shape[d] < 0 || (n.shape[d] > 0 && start + (n.shape[d] - 1) * step >= sn.shape[d]))
            err(BG_ERR_INVALID, "SLICE: range exceeds the input's extent");
        }
        kind_[i] = K_VIEW;
        break;
      }
      case BG_OP_REDUCE: case BG_OP_FUSED_SOFTMAX: case BG_OP_LAYER_NORM:
        kind_[i] = K_ROW;
        v.set_dense(n.shape, n.rank);
        v.slot = new_slot(n.numel() * dtype_size(n.dtype), false, i);
        break;
      case BG_OP_MATMUL: case BG_OP_INDEX: case BG_OP_CROSS_ENTROPY:
      case BG_OP_TRIL: case BG_OP_TRIU: case BG_OP_FLIP: case BG_OP_CONCAT: case BG_OP_CUMSUM:
      case BG_OP_SORT_INDICES: case BG_OP_TOPK_INDICES: case BG_OP_SCATTER:
        kind_[i] = K_OTHER;
        v.set_dense(n.shape, n.rank);
        v.slot = new_slot(n.numel() * dtype_size(n.dtype), false, i);
        break;
      default:
        if (!is_ew_op(n.op)) err(BG_ERR_UNSUPPORTED, std::string("opcode ") + op_name(n.op) + " is not supported by the CUDA bridge");
        kind_[i] = K_EW;
        v.set_dense(n.shape, n.rank);
        // every computed value gets a slot id up front so that views of it can name it; a slot
        // that no unit writes is never allocated
        v.slot = new_slot(n.numel() * dtype_size(n.dtype), false, i);
        break;
    }
  }
}

// Second half of view construction: needs to know which EW nodes are materialised, so it runs
// after `analyse` decided that every input of a VIEW node is materialised.
static bool reshape_view(const View& in, const int64_t* shp, int rank, View& out) {
  if (!in.contiguous()) return false;
  out = in;
  out.set_dense(shp, rank);
  return true;
}

void Compiler::analyse() {
  const int nn = (int)nodes_.size();
  cons_.assign(nn, {});
  for (int i = 0; i < nn; ++i)
    if (kind_[i] != K_DEAD)
      for (int in : nodes_[i].in) cons_[resolve(in)].push_back(i);
  // views (metadata only; a RESHAPE of a non-contiguous view becomes a copy unit)
  for (int i = 0; i < nn; ++i) {
    if (kind_[i] != K_VIEW) continue;
    Node& n = nodes_[i];
    const int src = resolve(n.in[0]);
    const View& sv = view_[src];
    if (n.dtype != sv.dtype) err(BG_ERR_INVALID, std::string(op_name(n.op)) + ": a view cannot change the dtype of its input (" +
                                                 dtype_name(sv.dtype) + " -> " + dtype_name(n.dtype) + ")");
    View v;
    if (n.op == BG_OP_PERMUTE) {
      v = sv;
      for (int d = 0; d < n.rank; ++d) { v.shape[d] = sv.shape[n.iarg[d]]; v.stride[d] = sv.stride[n.iarg[d]]; }
      leaflike_[i] = leaflike_[src];
    } else if (n.op == BG_OP_BROADCAST_TO) {
      v = sv;
      v.rank = n.rank;
      const int lead = n.rank - sv.rank;
      if (lead < 0) err(BG_ERR_INVALID, "BROADCAST_TO: rank shrinks");
      for (int d = 0; d < n.rank; ++d) {
        v.shape[d] = n.shape[d];
        if (d < lead) v.stride[d] = 0;
        else if (sv.shape[d - lead] == n.shape[d]) v.stride[d] = sv.stride[d - lead];
        else if (sv.shape[d - lead] == 1) v.stride[d] = 0;
        else err(BG_ERR_INVALID, "BROADCAST_TO: shapes are not broadcastable");
      }
      leaflike_[i] = leaflike_[src];
    } else if (n.op == BG_OP_SLICE) {
      if (sv.is_const) { v = sv; v.set_dense(n.shape, n.rank); leaflike_[i] = 1; }
      else {
        v = sv;
        for (int d = 0; d < n.rank; ++d) {
          const int64_t start = n.iarg[d] & (((int64_t)1 << 40) - 1), step = n.iarg[d] >> 40;
          v.off += start * sv.stride[d];
          v.stride[d] = sv.stride[d] * step;
          v.shape[d] = n.shape[d];
        }
        leaflike_[i] = leaflike_[src];
      }
    } else {  // RESHAPE
      if (nodes_[src].numel() != n.numel()) err(BG_ERR_INVALID, "RESHAPE: element count changes");
      if (sv.is_const) { v = sv; v.set_dense(n.shape, n.rank); leaflike_[i] = 1; }
      else if (reshape_view(sv, n.shape, n.rank, v)) leaflike_[i] = leaflike_[src];
      else {
        kind_[i] = K_OTHER;  // dense copy of the strided source, then a plain view of the copy
        copy_src_[i] = sv;
        v = View();
        v.set_dense(n.shape, n.rank);
        v.slot = new_slot(n.numel() * dtype_size(n.dtype), false, i);
        leaflike_[i] = 0;
      }
    }
    v.dtype = n.dtype;
    view_[i] = v;
  }
  // depth + grouping
  depth_.assign(nn, 0);
  group_.resize(nn);
  for (int i = 0; i < nn; ++i) group_[i] = i;
  auto same_shape = [&](int a, int b) {
    if (nodes_[a].rank != nodes_[b].rank) return false;
    for (int d = 0; d < nodes_[a].rank; ++d)
      if (nodes_[a].shape[d] != nodes_[b].shape[d]) return false;
    return true;
  };
  auto mergeable = [&](int n, int i) {
    return ctx_->fusion && kind_[i] == K_EW && kind_[n] == K_EW && same_shape(n, i) && !force_break_[i];
  };
  for (int i = 0; i < nn; ++i) {
    const Node& n = nodes_[i];
    int d = 0;
    if (kind_[i] == K_LEAF || kind_[i] == K_CONST) d = 0;
    else if (kind_[i] == K_ALIAS) d = depth_[n.in[0]];
    else if (kind_[i] == K_VIEW) { int s = resolve(n.in[0]); d = depth_[s]; }
    else if (kind_[i] == K_EW) {
      for (int in : n.in) {
        int s = resolve(in);
        int c = mergeable(i, s) ? depth_[s] : depth_[s] + (leaflike_[s] ? 0 : 1);
        d = std::max(d, c);
      }
    } else {
      for (int in : n.in) { int s = resolve(in); d = std::max(d, depth_[s] + (leaflike_[s] ? 0 : 1)); }
    }
    depth_[i] = d;
    if (kind_[i] == K_EW)
      for (int in : n.in) {
        int s = resolve(in);
        if (mergeable(i, s) && depth_[s] == d) group_[find(i)] = find(s);
      }
  }
  // tails
  tail_of_group_.assign(nn, -1);
  attached_.assign(nn, -1);
  if (ctx_->fusion)
    for (int i = 0; i < nn; ++i) {
      if (kind_[i] != K_ROW) continue;
      const int x = resolve(nodes_[i].in[0]);
      if (kind_[x] != K_EW || force_break_[x]) continue;
      int64_t rows, cols;
      View xin;
      bool trailing;
      if (!row_geometry(i, rows, cols, xin, trailing) || !trailing) continue;
      const int g = find(x);
      if (tail_of_group_[g] >= 0) continue;
      // layer norm weight/bias must not be produced inside the same group
      bool ok = true;
      for (size_t k = 1; k < nodes_[i].in.size(); ++k) {
        int w = resolve(nodes_[i].in[k]);
        if (kind_[w] == K_EW && find(w) == g) ok = false;
        if (depth_[w] + (leaflike_[w] ? 0 : 1) > depth_[x]) ok = false;
      }
      if (!ok) continue;
      tail_of_group_[g] = i;
      attached_[i] = g;
    }
  // materialisation
  need_mat_.assign(nn, 0);
  for (int i = 0; i < nn; ++i) {
    if (kind_[i] != K_EW) continue;
    if (i == root_) need_mat_[i] = 1;
    for (int c : cons_[i]) {
      if (kind_[c] == K_EW && find(c) == find(i)) continue;
      if (kind_[c] == K_ROW && attached_[c] == find(i) && resolve(nodes_[c].in[0]) == i) continue;
      need_mat_[i] = 1;
    }
  }
}

bool Compiler::row_geometry(int r, int64_t& rows, int64_t& cols, View& xin, bool& trailing) {
  const Node& n = nodes_[r];
  const int x = resolve(n.in[0]);
  const Node& xn = nodes_[x];
  xin = view_[x];
  trailing = false;
  if (n.op == BG_OP_LAYER_NORM) {
    rows = n.iarg[0];
    cols = n.iarg[1];
    if (rows * cols != xn.numel() || n.in.size() != 3) err(BG_ERR_INVALID, "LAYER_NORM: rows x cols does not match the input");
    trailing = true;
    return true;
  }
  if (n.op == BG_OP_FUSED_SOFTMAX) {
    int64_t axis = n.iarg[0];
    if (axis < 0 || axis >= xn.rank) err(BG_ERR_INVALID, "FUSED_SOFTMAX: axis out of range");
    int64_t inner = 1;
    for (int d = (int)axis + 1; d < xn.rank; ++d) inner *= xn.shape[d];
    cols = xn.shape[axis];
    rows = cols ? xn.numel() / cols : 0;
    trailing = inner == 1;
    return true;
  }
  // REDUCE
  const uint64_t mask = (uint64_t)n.iarg[1];
  int k = xn.rank;
  while (k > 0 && ((mask >> (k - 1)) & 1)) --k;
  bool tr = true;
  for (int d = 0; d < k; ++d)
    if ((mask >> d) & 1) tr = false;
  cols = 1;
  rows = 1;
  for (int d = 0; d < xn.rank; ++d) {
    if ((mask >> d) & 1) cols *= xn.shape[d]; else rows *= xn.shape[d];
  }
  trailing = tr;
  return true;
}

// ---------------------------------------------------------------------------------------
// Program construction
// ---------------------------------------------------------------------------------------
struct VInstr {
  uint8_t op, type;
  int dst, a, b, c;
  uint16_t aux;
};

static std::string gelu_expr_text();

bool Compiler::build_program(const std::vector<int>& members, int tail_node, ProgramSpec& ps, std::vector<int>& dep_nodes,
                             std::vector<int>& out_nodes, std::string& why) {
  std::vector<VInstr> code;
  int next_v = 0;
  std::map<int, int> vreg;                        // node -> vreg (natural class)
  std::map<std::pair<int, int>, int> cvt_memo;    // (vreg, class) -> vreg
  std::map<int, int> load_memo;                   // external node -> vreg
  std::vector<View> in_views;
  std::vector<int> in_nodes;
  std::vector<int64_t> consts;
  std::set<int> member_set(members.begin(), members.end());
  const Node& lead = nodes_[tail_node >= 0 ? resolve(nodes_[tail_node].in[0]) : members[0]];
  // iteration shape = shape of the member nodes (all equal); for a standalone tail, the input's.
  int it_rank = lead.rank;
  int64_t it_shape[kMaxRank];
  for (int d = 0; d < it_rank; ++d) it_shape[d] = lead.shape[d];

  auto add_input = [&](int node, const View& v) -> int {
    if ((int)in_views.size() >= kEwMaxInputs) return -1;
    in_views.push_back(v);
    in_nodes.push_back(node);
    return (int)in_views.size() - 1;
  };
  auto add_const = [&](int64_t bits) -> int {
    for (size_t i = 0; i < consts.size(); ++i)
      if (consts[i] == bits) return (int)i;
    if ((int)consts.size() >= kEwMaxConsts) return -1;
    consts.push_back(bits);
    return (int)consts.size() - 1;
  };
  bool failed = false;
  auto emit = [&](uint8_t op, uint8_t type, int a, int b, int c, uint16_t aux) -> int {
    int d = next_v++;
    code.push_back({op, type, d, a, b, c, aux});
    return d;
  };
  auto operand = [&](int node, EwType want) -> int {
    node = resolve(node);
    int v, c;
    const View& vw = view_[node];
    if (member_set.count(node)) {
      v = vreg[node];
      c = cls_of(nodes_[node].dtype);
    } else if (vw.is_const) {
      // a constant is emitted directly in the class its consumer computes in: that is the value
      // NumPy's promotion (or an explicit CAST) would have produced
      const EwType nat = cls_of(vw.dtype);
      const bool want_f = want == T_F32 || want == T_F64;
      int64_t bits;
      EwType cc;
      if (nat == T_F32 || nat == T_F64) {
        double dv = nat == T_F32 ? (double)(float)vw.cf : vw.cf;
        cc = want_f ? want : nat;
        if (cc == T_F32) dv = (double)(float)dv;
        memcpy(&bits, &dv, 8);
      } else if (want_f) {
        double dv = (double)vw.ci;
        cc = want;
        memcpy(&bits, &dv, 8);
      } else {
        cc = (nat == T_B && want == T_I64) ? T_I64 : nat;
        bits = nat == T_B ? (vw.ci != 0) : vw.ci;
      }
      int ci = add_const(bits);
      if (ci < 0) { failed = true; why = "too many constants"; return 0; }
      auto key = std::make_pair(-1000 - ci, (int)cc);
      auto it = cvt_memo.find(key);
      if (it != cvt_memo.end()) v = it->second;
      else { v = emit(E_CONST, cc, 0, 0, 0, (uint16_t)ci); cvt_memo[key] = v; }
      c = cc;
    } else {
      auto it = load_memo.find(node);
      if (it != load_memo.end()) v = it->second;
      else {
        int idx = add_input(node, vw);
        if (idx < 0) { failed = true; why = "too many inputs"; return 0; }
        v = emit(E_LOAD, cls_of(vw.dtype), 0, 0, 0, (uint16_t)idx);
        load_memo[node] = v;
      }
      c = cls_of(vw.dtype);
    }
    if (c == (int)want) return v;
    auto key = std::make_pair(v, (int)want);
    auto it = cvt_memo.find(key);
    if (it != cvt_memo.end()) return it->second;
    int r = emit(E_CVT, want, v, 0, 0, (uint16_t)c);
    cvt_memo[key] = r;
    return r;
  };

  for (int m : members) {
    const Node& n = nodes_[m];
    const EwType nc = cls_of(n.dtype);
    int r = -1;
    auto need = [&](size_t k) {
      if (n.in.size() != k) err(BG_ERR_INVALID, std::string(op_name(n.op)) + ": expected " + std::to_string(k) + " inputs");
    };
    // The float64 tanh GELU of an fp32 value, in a plan whose leaves hold no float64 data, is evaluated in fp32 and
    // widened (the same rule sends such contractions to the 3xTF32 path).  The float64 instructions already emitted
    // for its inner nodes die below unless something else reads them.
    if (n.op == BG_OP_MUL && n.dtype == BG_F64 && n.in.size() == 2 && ctx_->fusion &&
        (ctx_->f64_mode == 1 || (ctx_->f64_mode == 2 && !has_f64_leaf_))) {
      int x = -1;
      for (int k = 0; k < 2 && x < 0; ++k) {
        const int h = resolve(n.in[k]);
        if (kind_[h] != K_EW || nodes_[h].op != BG_OP_MUL || nodes_[h].in.size() != 2) continue;
        for (int j = 0; j < 2; ++j) {
          const int c = resolve(nodes_[h].in[j]);
          if (kind_[c] == K_CONST && view_[c].is_const && dtype_is_float(nodes_[c].dtype) && view_[c].cf == 0.5) x = resolve(nodes_[h].in[1 - j]);
        }
      }
      if (x >= 0 && nodes_[x].dtype == BG_F32 && act_expr(m, x, find(m), 0) == gelu_expr_text()) {
        const int xv = operand(x, T_F32);
        if (failed) return false;
        const int y = emit(E_GELU, T_F32, xv, 0, 0, 0);
        vreg[m] = emit(E_CVT, T_F64, y, 0, 0, (uint16_t)T_F32);
        continue;
      }
    }
    switch (n.op) {
      case BG_OP_ADD: case BG_OP_MUL: case BG_OP_DIV: {
        need(2);
        int a = operand(n.in[0], nc), b = operand(n.in[1], nc);
        uint8_t op = n.op == BG_OP_ADD ? E_ADD : (n.op == BG_OP_MUL ? E_MUL : E_DIV);
        if (nc == T_B) {
          if (n.op == BG_OP_DIV) err(BG_ERR_UNSUPPORTED, "DIV on bool tensors is not supported");
          op = n.op == BG_OP_ADD ? E_OR : E_AND;
        }
        r = emit(op, nc, a, b, 0, 0);
        break;
      }
      case BG_OP_NEG: case BG_OP_EXP: case BG_OP_LOG: case BG_OP_ABS: case BG_OP_SIGN: case BG_OP_SIN: case BG_OP_COS: {
        need(1);
        if (nc == T_B) err(BG_ERR_UNSUPPORTED, std::string(op_name(n.op)) + " on bool tensors is not supported");
        const bool transcend = n.op == BG_OP_EXP || n.op == BG_OP_LOG || n.op == BG_OP_SIN || n.op == BG_OP_COS;
        if (nc == T_I64 && transcend) err(BG_ERR_UNSUPPORTED, std::string(op_name(n.op)) + " on integer tensors is not supported");
        int a = operand(n.in[0], nc);
        uint8_t op = E_NEG;
        switch (n.op) {
          case BG_OP_EXP: op = E_EXP; break;
          case BG_OP_LOG: op = E_LOG; break;
          case BG_OP_ABS: op = E_ABS; break;
          case BG_OP_SIGN: op = E_SIGN; break;
          case BG_OP_SIN: op = E_SIN; break;
          case BG_OP_COS: op = E_COS; break;
        }
        r = emit(op, nc, a, 0, 0, 0);
        break;
      }
      case BG_OP_ISNAN: {
        need(1);
        EwType ic = cls_of(nodes_[resolve(n.in[0])].dtype);
        int a = operand(n.in[0], ic);
        r = emit(E_ISNAN, ic, a, 0, 0, 0);
        break;
      }
      case BG_OP_CMP: {
        need(2);
        int pd = promote(nodes_[resolve(n.in[0])].dtype, nodes_[resolve(n.in[1])].dtype);
        EwType pc = cls_of(pd);
        int a = operand(n.in[0], pc), b = operand(n.in[1], pc);
        if (n.iarg[0] < 0 || n.iarg[0] > 5) err(BG_ERR_INVALID, "CMP: unknown comparison");
        r = emit(E_CMP, pc, a, b, 0, (uint16_t)n.iarg[0]);
        break;
      }
      case BG_OP_WHERE: {
        need(3);
        int c = operand(n.in[0], T_B), a = operand(n.in[1], nc), b = operand(n.in[2], nc);
        r = emit(E_WHERE, nc, c, a, b, 0);
        break;
      }
      case BG_OP_CAST: {
        need(1);
        int a = operand(n.in[0], nc);
        // a CAST between dtypes of one class still needs its own register only when it narrows
        r = narrow_dtype(n.dtype) ? emit(E_NARROW, nc, a, 0, 0, (uint16_t)n.dtype) : a;
        break;
      }
      default:
        err(BG_ERR_UNSUPPORTED, std::string("opcode ") + op_name(n.op) + " inside an elementwise group");
    }
    if (failed) return false;
    if (n.op != BG_OP_CAST && narrow_dtype(n.dtype) && nc != T_B) r = emit(E_NARROW, nc, r, 0, 0, (uint16_t)n.dtype);
    vreg[m] = r;
  }
  // outputs
  std::vector<int> out_list;
  for (int m : members)
    if (need_mat_[m]) out_list.push_back(m);
  int tail_reg_v = -1;
  EwProgram& P = ps.prog;
  memset(&P, 0, sizeof(P));
  int n_out = 0;
  for (int m : out_list) {
    if (n_out >= kEwMaxOutputs) { why = "too many outputs"; return false; }
    own_slot(m);
    code.push_back({E_STORE, (uint8_t)cls_of(nodes_[m].dtype), -1, vreg[m], 0, 0, (uint16_t)n_out});
    P.outputs[n_out].dtype = nodes_[m].dtype;
    ps.out_slot[n_out] = view_[m].slot;
    out_nodes.push_back(m);
    ++n_out;
  }
  int64_t rows = 0, cols = 0;
  if (tail_node >= 0) {
    const Node& t = nodes_[tail_node];
    View xin;
    bool trailing;
    row_geometry(tail_node, rows, cols, xin, trailing);
    const int x = resolve(t.in[0]);
    EwType xc = cls_of(nodes_[x].dtype);
    EwType want = xc;
    if (t.op == BG_OP_FUSED_SOFTMAX) {
      if (xc != T_F32 && xc != T_F64) err(BG_ERR_UNSUPPORTED, "FUSED_SOFTMAX on non-float tensors");
    } else if (t.op == BG_OP_LAYER_NORM) {
      if (xc != T_F32 && xc != T_F64) err(BG_ERR_UNSUPPORTED, "LAYER_NORM on non-float tensors");
    } else {
      const int rop = (int)t.iarg[0];
      if (rop < 0 || rop > BG_RED_PROD) err(BG_ERR_INVALID, "REDUCE: unknown reduction");
      if (rop == BG_RED_PROD && nodes_[x].dtype != BG_F32 && nodes_[x].dtype != BG_F64 && nodes_[x].dtype != BG_I64) err(BG_ERR_UNSUPPORTED, "REDUCE prod: float32, float64 and int64 only");
      if (rop == BG_RED_ANY || rop == BG_RED_ALL) want = T_B;
      else if (xc == T_B) want = T_I64;
    }
    tail_reg_v = operand(x, want);
    if (failed) return false;
    if (n_out >= kEwMaxOutputs) { why = "too many outputs"; return false; }
    own_slot(tail_node);
    P.outputs[n_out].dtype = t.dtype;
    ps.out_slot[n_out] = view_[tail_node].slot;
    out_nodes.push_back(tail_node);
    P.tail_out = n_out;
    P.tail_out_dtype = t.dtype;
    P.tail_type = want;
    ++n_out;
    if (t.op == BG_OP_FUSED_SOFTMAX) P.tail = TAIL_SOFTMAX;
    else if (t.op == BG_OP_LAYER_NORM) {
      P.tail = TAIL_LAYERNORM;
      P.tail_eps = (float)t.farg[0];
      for (int k = 1; k <= 2; ++k) {
        int w = resolve(t.in[k]);
        const View& wv = view_[w];
        if (wv.is_const || !wv.contiguous() || wv.numel() != cols || !dtype_is_float(wv.dtype))
          err(BG_ERR_UNSUPPORTED, "LAYER_NORM: weight and bias must be dense float vectors of `cols` elements");
        int idx = add_input(w, wv);
        if (idx < 0) { why = "too many inputs"; return false; }
        if (k == 1) P.tail_w = idx; else P.tail_b = idx;
      }
    } else {
      P.tail = TAIL_REDUCE;
      P.tail_arg = (int)t.iarg[0];
    }
    P.rows = rows;
    P.cols = cols;
  }
  // iteration space: collapse dims that every operand walks contiguously
  int64_t numel = 1;
  for (int d = 0; d < it_rank; ++d) numel *= it_shape[d];
  std::vector<std::vector<int64_t>> strides(in_views.size(), std::vector<int64_t>(it_rank, 0));
  const int n_ew_inputs = (int)in_views.size();
  for (int k = 0; k < n_ew_inputs; ++k) {
    if (tail_node >= 0 && P.tail == TAIL_LAYERNORM && (k == P.tail_w || k == P.tail_b)) continue;
    const View& v = in_views[k];
    const int lead_d = it_rank - v.rank;
    if (lead_d < 0) err(BG_ERR_INVALID, "elementwise operand has higher rank than the result");
    for (int d = 0; d < it_rank; ++d) {
      if (d < lead_d) { strides[k][d] = 0; continue; }
      int64_t e = v.shape[d - lead_d];
      if (e == it_shape[d]) strides[k][d] = e == 1 ? 0 : v.stride[d - lead_d];
      else if (e == 1) strides[k][d] = 0;
      else err(BG_ERR_INVALID, "elementwise operand shape is not broadcastable to the result");
    }
  }
  std::vector<int64_t> cshape;
  std::vector<std::vector<int64_t>> cstr(in_views.size());
  for (int d = 0; d < it_rank; ++d) {
    if (it_shape[d] == 1) continue;
    bool merge = !cshape.empty();
    if (merge)
      for (int k = 0; k < n_ew_inputs; ++k) {
        if (cstr[k].empty()) continue;
        if (cstr[k].back() != strides[k][d] * it_shape[d]) { merge = false; break; }
      }
    if (merge) {
      cshape.back() *= it_shape[d];
      for (int k = 0; k < n_ew_inputs; ++k)
        if (!cstr[k].empty()) cstr[k].back() = strides[k][d];
    } else {
      cshape.push_back(it_shape[d]);
      for (int k = 0; k < n_ew_inputs; ++k) cstr[k].push_back(strides[k][d]);
    }
  }
  if (cshape.empty()) {
    cshape.push_back(1);
    for (int k = 0; k < n_ew_inputs; ++k) cstr[k].assign(1, 0);
  }
  if ((int)cshape.size() > kEwMaxDims) { why = "iteration space has too many non-collapsible dimensions"; return false; }
  P.ndim = (int)cshape.size();
  for (int d = 0; d < P.ndim; ++d) P.shape[d] = cshape[d];
  P.numel = numel;
  if (tail_node < 0) { P.rows = 0; P.cols = 0; }
  const bool row_vec = tail_node < 0 || (cols % 4 == 0);
  P.n_inputs = n_ew_inputs;
  for (int k = 0; k < n_ew_inputs; ++k) {
    const View& v = in_views[k];
    EwOperand& o = P.inputs[k];
    o.dtype = v.dtype;
    ps.in_slot[k] = v.slot;
    ps.in_off_bytes[k] = v.off * dtype_size(v.dtype);
    dep_nodes.push_back(in_nodes[k]);
    if (tail_node >= 0 && P.tail == TAIL_LAYERNORM && (k == P.tail_w || k == P.tail_b)) { o.mode = A_CONTIG; continue; }
    bool all_zero = true, contig = true;
    int64_t expect = 1;
    for (int d = P.ndim - 1; d >= 0; --d) {
      o.stride[d] = cstr[k][d];
      if (cstr[k][d] != 0) all_zero = false;
      if (cstr[k][d] != expect) contig = false;
      expect *= cshape[d];
    }
    if (numel <= 1) { all_zero = true; }
    o.mode = all_zero ? A_SCALAR : (contig ? A_CONTIG : A_STRIDED);
    const int es = dtype_size(v.dtype);
    const int64_t vec_bytes = std::min<int64_t>(16, 4 * es);
    bool ok = (ps.in_off_bytes[k] % vec_bytes) == 0 && row_vec;
    if (o.mode == A_STRIDED) {
      for (int d = 0; d + 1 < P.ndim; ++d)
        if (o.stride[d] % 4 != 0) ok = false;
    }
    o.vec_ok = ok ? 1 : 0;
  }
  P.n_outputs = n_out;
  for (int k = 0; k < n_out; ++k) P.outputs[k].vec_ok = row_vec ? 1 : 0;
  P.n_consts = (int)consts.size();
  for (size_t k = 0; k < consts.size(); ++k) P.consts[k] = consts[k];
  // ---- peephole pass (fp32): super-instructions and direct global operands -----------------
  {
    auto is_unary = [](uint8_t op) {
      return op == E_NEG || op == E_EXP || op == E_LOG || op == E_ABS || op == E_SIGN || op == E_SIN || op == E_COS ||
             op == E_ISNAN || op == E_CVT || op == E_NARROW || op == E_STORE || op == E_RELU || op == E_EXPNEG || op == E_COPY ||
             op == E_GELU;
    };
    auto n_src = [&](const VInstr& I) { return (I.op == E_LOAD || I.op == E_CONST) ? 0 : (is_unary(I.op) ? 1 : (I.op == E_WHERE ? 3 : 2)); };
    auto src = [](VInstr& I, int k) -> int& { return k == 0 ? I.a : (k == 1 ? I.b : I.c); };
    std::vector<char> dead(code.size(), 0);
    auto recount = [&](std::vector<int>& uses, std::vector<int>& def) {
      uses.assign(next_v, 0);
      def.assign(next_v, -1);
      for (size_t i = 0; i < code.size(); ++i) {
        if (dead[i]) continue;
        VInstr& I = code[i];
        for (int k = 0; k < n_src(I); ++k)
          if (src(I, k) >= 0) uses[src(I, k)]++;
        if (I.dst >= 0) def[I.dst] = (int)i;
      }
      if (tail_reg_v >= 0) uses[tail_reg_v] += 2;
    };
    std::vector<int> uses, def;
    recount(uses, def);
    // values nothing reads (the inner nodes of an expression that was replaced as a whole)
    for (bool again = true; again;) {
      again = false;
      for (size_t i = code.size(); i-- > 0;) {
        if (dead[i] || code[i].op == E_STORE || code[i].dst < 0 || uses[code[i].dst] != 0) continue;
        dead[i] = 1;
        again = true;
      }
      if (again) recount(uses, def);
    }
    // an fp32 value widened only to be stored into a float64 output is stored by the fp32 instruction itself
    for (size_t i = 0; i < code.size(); ++i) {
      if (dead[i]) continue;
      VInstr& S = code[i];
      if (S.op != E_STORE || S.type != T_F64 || S.a < 0 || def[S.a] < 0 || uses[S.a] != 1 || S.a == tail_reg_v) continue;
      const int wi = def[S.a];
      const VInstr& W = code[wi];
      if (W.op != E_CVT || W.type != T_F64 || (W.aux & 0xF) != T_F32) continue;
      if (P.outputs[S.aux].dtype != BG_F64 || !P.outputs[S.aux].vec_ok) continue;
      S.type = T_F32;
      S.a = W.a;
      dead[wi] = 1;
      recount(uses, def);
    }
    for (size_t i = 0; i < code.size(); ++i) {
      if (dead[i]) continue;
      VInstr& I = code[i];
      if (I.type != T_F32) continue;
      if (I.op == E_WHERE && I.a >= 0 && I.b >= 0 && I.c >= 0 && def[I.a] >= 0 && def[I.c] >= 0) {
        VInstr& C = code[def[I.a]];
        VInstr& Z = code[def[I.c]];
        if (C.op == E_CMP && C.type == T_F32 && C.aux == BG_CMP_GT && C.a == I.b && C.b == I.c && uses[I.a] == 1 &&
            Z.op == E_CONST && Z.type == T_F32 && consts[Z.aux] == 0) {
          dead[def[I.a]] = 1;
          I.op = E_RELU;
          I.a = I.b;
          I.b = I.c = 0;
          recount(uses, def);
        }
      } else if (I.op == E_EXP && I.a >= 0 && def[I.a] >= 0) {
        VInstr& N = code[def[I.a]];
        if (N.op == E_NEG && N.type == T_F32 && uses[I.a] == 1) {
          dead[def[I.a]] = 1;
          I.op = E_EXPNEG;
          I.a = N.a;
          recount(uses, def);
        }
      } else if (I.op == E_ADD && I.a >= 0 && I.b >= 0) {
        for (int k = 1; k >= 0; --k) {
          int v = k ? I.b : I.a;
          if (def[v] < 0) continue;
          VInstr& N = code[def[v]];
          if (N.op == E_NEG && N.type == T_F32 && uses[v] == 1) {
            int other = k ? I.a : I.b;
            dead[def[v]] = 1;
            I.op = E_SUB;
            I.a = other;
            I.b = N.a;
            recount(uses, def);
            break;
          }
        }
      }
    }
    // fp32 constants become operands of the fp32 instructions that read them; single-use dense fp32
    // LOADs become direct operands of their consumer
    auto f32_value_op = [](uint8_t op) {
      return op == E_ADD || op == E_SUB || op == E_MUL || op == E_DIV || op == E_NEG || op == E_EXP || op == E_LOG ||
             op == E_ABS || op == E_SIGN || op == E_SIN || op == E_COS || op == E_RELU || op == E_EXPNEG || op == E_GELU;
    };
    auto dense_f32_in = [&](int k) {
      const EwOperand& o = P.inputs[k];
      return o.mode == A_CONTIG && o.dtype == BG_F32 && o.vec_ok;
    };
    for (size_t i = 0; i < code.size(); ++i) {
      if (dead[i]) continue;
      VInstr& I = code[i];
      if (I.type != T_F32) continue;
      const bool arith = f32_value_op(I.op);
      if (!arith && I.op != E_CMP && I.op != E_WHERE) continue;
      for (int k = (I.op == E_WHERE ? 1 : 0); k < n_src(I); ++k) {
        int v = src(I, k);
        if (v < 0 || def[v] < 0) continue;
        VInstr& L = code[def[v]];
        if (L.op == E_CONST && L.type == T_F32) {
          src(I, k) = -3000 - (int)L.aux;
          continue;
        }
        if (uses[v] != 1 || L.op != E_LOAD || L.type != T_F32 || !dense_f32_in(L.aux)) continue;
        dead[def[v]] = 1;
        src(I, k) = -1000 - (int)L.aux;
      }
    }
    recount(uses, def);
    // constants nobody reads any more
    for (size_t i = 0; i < code.size(); ++i)
      if (!dead[i] && code[i].op == E_CONST && uses[code[i].dst] == 0) dead[i] = 1;
    // a final STORE of a value produced by fp32 arithmetic becomes that instruction's destination
    for (size_t i = 0; i < code.size(); ++i) {
      if (dead[i]) continue;
      VInstr& S = code[i];
      if (S.op != E_STORE || S.type != T_F32 || S.a < 0 || def[S.a] < 0) continue;
      if (uses[S.a] != 1 || S.a == tail_reg_v) continue;
      const EwOutput& o = P.outputs[S.aux];
      if ((o.dtype != BG_F32 && o.dtype != BG_F64) || !o.vec_ok) continue;   // float64: the store widens
      VInstr& D = code[def[S.a]];
      if (D.type != T_F32 || !(f32_value_op(D.op) || D.op == E_WHERE)) continue;
      D.dst = -2000 - (int)S.aux;
      dead[i] = 1;
    }
    // what is left of the dense fp32 LOADs and STOREs runs as a copy on the fast path
    for (size_t i = 0; i < code.size(); ++i) {
      if (dead[i]) continue;
      VInstr& I = code[i];
      if (I.type != T_F32) continue;
      if (I.op == E_LOAD && dense_f32_in(I.aux)) {
        I.op = E_COPY;
        I.a = -1000 - (int)I.aux;
        I.aux = 0;
      } else if (I.op == E_STORE && (P.outputs[I.aux].dtype == BG_F32 || P.outputs[I.aux].dtype == BG_F64) && P.outputs[I.aux].vec_ok) {
        I.op = E_COPY;
        I.dst = -2000 - (int)I.aux;
        I.aux = 0;
      }
    }
    std::vector<VInstr> kept;
    for (size_t i = 0; i < code.size(); ++i)
      if (!dead[i]) kept.push_back(code[i]);
    code.swap(kept);
    dead.assign(code.size(), 0);
    recount(uses, def);
    // a value whose only reader is the next instruction stays in the accumulator (-4000)
    for (size_t i = 0; i + 1 < code.size(); ++i) {
      VInstr& Pd = code[i];
      VInstr& C = code[i + 1];
      if (Pd.type != T_F32 || C.type != T_F32 || Pd.dst < 0 || uses[Pd.dst] != 1) continue;
      if (!(f32_value_op(Pd.op) || Pd.op == E_WHERE)) continue;
      const int v = Pd.dst;
      bool ok = false;
      if (C.op == E_ADD || C.op == E_MUL) {
        // c = 1 records the exchange for readers that want the operands in graph order
        if (C.b == v && C.a != v) { std::swap(C.a, C.b); C.c = 1; }
        ok = C.a == v;
      } else if (C.op == E_SUB || C.op == E_DIV || C.op == E_CMP) {
        ok = C.a == v && C.b != v;
      } else if (C.op == E_WHERE) {
        ok = C.b == v && C.a != v && C.c != v;
      } else if (C.op == E_COPY || (f32_value_op(C.op) && is_unary(C.op))) {
        ok = C.a == v;
      }
      if (!ok) continue;
      Pd.dst = -4000;
      if (C.op == E_WHERE) C.b = -4000;
      else C.a = -4000;
    }
  }
  if ((int)code.size() > kEwMaxInstr) { why = "too many instructions"; return false; }
  // register allocation (linear scan; a destination may take over a source that dies here)
  std::vector<int> last(next_v, -1);
  for (size_t i = 0; i < code.size(); ++i) {
    const VInstr& I = code[i];
    auto use = [&](int v) { if (v >= 0) last[v] = (int)i; };
    const bool unary = I.op == E_NEG || I.op == E_EXP || I.op == E_LOG || I.op == E_ABS || I.op == E_SIGN || I.op == E_SIN ||
                       I.op == E_COS || I.op == E_ISNAN || I.op == E_CVT || I.op == E_NARROW || I.op == E_STORE ||
                       I.op == E_RELU || I.op == E_EXPNEG || I.op == E_COPY || I.op == E_GELU;
    if (I.op == E_LOAD || I.op == E_CONST) continue;
    use(I.a);
    if (!unary) use(I.b);
    if (I.op == E_WHERE) use(I.c);
  }
  if (tail_reg_v >= 0) last[tail_reg_v] = (int)code.size() + 1;
  std::vector<int> phys(next_v, -1);
  std::vector<char> busy;
  auto alloc_reg = [&]() {
    for (size_t i = 0; i < busy.size(); ++i)
      if (!busy[i]) { busy[i] = 1; return (int)i; }
    busy.push_back(1);
    return (int)busy.size() - 1;
  };
  bool wide = false;
  P.n_instr = (int)code.size();
  for (size_t i = 0; i < code.size(); ++i) {
    const VInstr& I = code[i];
    EwInstr& O = P.instr[i];
    O.op = I.op;
    O.type = I.type;
    O.aux = I.aux;
    const bool unary = I.op == E_NEG || I.op == E_EXP || I.op == E_LOG || I.op == E_ABS || I.op == E_SIGN || I.op == E_SIN ||
                       I.op == E_COS || I.op == E_ISNAN || I.op == E_CVT || I.op == E_NARROW || I.op == E_STORE ||
                       I.op == E_RELU || I.op == E_EXPNEG || I.op == E_COPY || I.op == E_GELU;
    const bool leaf = I.op == E_LOAD || I.op == E_CONST;
    int srcs[3] = {leaf ? -1 : I.a, (leaf || unary) ? -1 : I.b, I.op == E_WHERE ? I.c : -1};
    auto enc = [&](int v) -> uint8_t {
      if (v == -4000) return kEwAcc;
      if (v <= -3000) return (uint8_t)(kEwConst | (-3000 - v));                 // constant operand
      if (v <= -1000 && v > -2000) return (uint8_t)(kEwDirect | (-1000 - v));   // direct global input
      return v >= 0 ? (uint8_t)phys[v] : 0;
    };
    O.a = enc(srcs[0]);
    O.b = enc(srcs[1]);
    O.c = enc(srcs[2]);
    if ((I.op == E_ADD || I.op == E_MUL) && I.type == T_F32 && I.c == 1) O.c = 1;   // operands were exchanged
    for (int k = 0; k < 3; ++k)
      if (srcs[k] >= 0 && last[srcs[k]] == (int)i && phys[srcs[k]] >= 0) {
        bool dup = false;
        for (int j = 0; j < k; ++j) dup |= srcs[j] == srcs[k];
        if (!dup) busy[phys[srcs[k]]] = 0;
      }
    if (I.type == T_F64 || I.type == T_I64) wide = true;
    if (I.op == E_CVT && ((I.aux & 0xF) == T_F64 || (I.aux & 0xF) == T_I64)) wide = true;
    if (I.dst == -4000) O.dst = kEwAcc;
    else if (I.dst <= -2000) O.dst = (uint8_t)(kEwDirect | (-2000 - I.dst));   // direct global output
    if (I.dst >= 0) {
      phys[I.dst] = alloc_reg();
      O.dst = (uint8_t)phys[I.dst];
      if (last[I.dst] < 0) busy[phys[I.dst]] = 0;
    }
  }
  if (busy.size() > 120) { why = "too many live registers"; return false; }
  P.n_regs = std::max<int>(1, (int)busy.size());
  P.wide = wide ? 1 : 0;
  if (tail_reg_v >= 0) P.tail_reg = phys[tail_reg_v];
  P.tail_acc = 0;
  if (tail_reg_v >= 0 && !code.empty()) {
    const VInstr& L = code.back();
    const bool value_op = L.op == E_ADD || L.op == E_SUB || L.op == E_MUL || L.op == E_DIV || L.op == E_NEG || L.op == E_EXP ||
                          L.op == E_LOG || L.op == E_ABS || L.op == E_SIGN || L.op == E_SIN || L.op == E_COS || L.op == E_RELU ||
                          L.op == E_EXPNEG || L.op == E_WHERE || L.op == E_COPY || L.op == E_GELU;
    if (L.type == T_F32 && value_op && L.dst == tail_reg_v) P.tail_acc = 1;
  }
  const int64_t per_chunk = (int64_t)P.n_regs * (wide ? 2 : 1) * 4096;
  if (per_chunk > 190 * 1024) { why = "register file does not fit shared memory"; return false; }
  ps.row = tail_node >= 0;
  if (ps.row && P.tail != TAIL_REDUCE) {
    const int64_t chunks = (cols + 1023) / 1024;
    if (chunks > rowwise_max_chunks(P.n_regs, P.wide)) { why = "row does not fit the on-chip register file"; return false; }
  }
  return true;
}

// Expression of an all-fp32 single-result program as text, e.g. "mul(relu(add(mul(i0,i1),i2)),expneg(i3))".
// Empty when the program is not a pure fp32 expression over dense vector-aligned operands.
static std::string program_signature(const EwProgram& P, int* kind, int* arg) {
  std::map<int, std::string> reg;
  std::string result;
  int n_results = 0;
  auto opname = [](int op) -> const char* {
    switch (op) {
      case E_ADD: return "add"; case E_SUB: return "sub"; case E_MUL: return "mul"; case E_DIV: return "div";
      case E_NEG: return "neg"; case E_EXP: return "exp"; case E_LOG: return "log"; case E_RELU: return "relu";
      case E_EXPNEG: return "expneg"; case E_ABS: return "abs";
    }
    return nullptr;
  };
  auto dense = [&](int k) {
    const EwOperand& o = P.inputs[k];
    return o.mode == A_CONTIG && o.dtype == BG_F32 && o.vec_ok;
  };
  bool ok = true;
  auto operand = [&](uint8_t r) -> std::string {
    if (r & kEwDirect) {
      if ((r & kEwConst) == kEwConst || !dense(r & 0x3f)) { ok = false; return "?"; }
      return "i" + std::to_string(r & 0x3f);
    }
    auto it = reg.find(r);
    if (it == reg.end()) { ok = false; return "?"; }
    return it->second;
  };
  for (int i = 0; i < P.n_instr && ok; ++i) {
    const EwInstr& I = P.instr[i];
    if (I.type != T_F32) return "";
    std::string v;
    if (I.op == E_LOAD) {
      if (!dense(I.aux)) return "";
      v = "i" + std::to_string(I.aux);
    } else if (I.op == E_STORE) {
      if (P.outputs[I.aux].dtype != BG_F32 || !P.outputs[I.aux].vec_ok) return "";
      result = operand(I.a);
      ++n_results;
      continue;
    } else if (I.op == E_COPY) {
      v = operand(I.a);
    } else {
      const char* nm = opname(I.op);
      if (!nm) return "";
      const bool binary = I.op == E_ADD || I.op == E_SUB || I.op == E_MUL || I.op == E_DIV;
      const bool exchanged = (I.op == E_ADD || I.op == E_MUL) && I.c == 1;
      v = std::string(nm) + "(" + operand(exchanged ? I.b : I.a) + (binary ? "," + operand(exchanged ? I.a : I.b) : "") + ")";
    }
    if (I.dst & kEwDirect) {
      if (P.outputs[I.dst & 0x7f].dtype != BG_F32 || !P.outputs[I.dst & 0x7f].vec_ok) return "";
      result = v;
      ++n_results;
    } else {
      reg[I.dst] = v;
    }
  }
  if (!ok) return "";
  if (P.tail == TAIL_NONE) {
    if (n_results != 1 || P.n_outputs != 1) return "";
    *kind = SK_FLAT;
    return result;
  }
  if (n_results != 0 || P.n_outputs != 1 || P.tail_type != T_F32 || P.tail_out_dtype != BG_F32) return "";
  auto it = reg.find(P.tail_reg);
  if (it == reg.end()) return "";
  if (P.tail == TAIL_SOFTMAX) { *kind = SK_SOFTMAX; return it->second; }
  if (P.tail == TAIL_REDUCE && (P.tail_arg == BG_RED_SUM || P.tail_arg == BG_RED_MEAN)) {
    *kind = SK_ROWSUM;
    *arg = P.tail_arg == BG_RED_MEAN;
    return it->second;
  }
  return "";
}

// A layer-norm row program whose row value is a plain sum of loaded operands (residual adds and a
// bias vector) runs in the specialised kernel.  Fills ps.ln_* and returns true when it matches.
static bool match_static_ln(ProgramSpec& ps) {
  const EwProgram& P = ps.prog;
  if (P.tail != TAIL_LAYERNORM || !static_ln_shape_ok(P.rows, P.cols)) return false;
  if (P.tail_type != T_F32 && P.tail_type != T_F64) return false;
  if (P.n_outputs < 1 || P.n_outputs > 2) return false;
  const bool wide = P.tail_type == T_F64;
  const int sum_dtype = wide ? BG_F64 : BG_F32;
  if (P.tail_out_dtype != BG_F32 && P.tail_out_dtype != BG_F64) return false;
  auto float_vec = [&](int k) {
    const EwOperand& o = P.inputs[k];
    return (o.dtype == BG_F32 || o.dtype == BG_F64) && ps.in_off_bytes[k] % 32 == 0;
  };
  if (!float_vec(P.tail_w) || !float_vec(P.tail_b)) return false;
  // 1 = dense rows, 2 = one vector for every row, 0 = neither
  auto half_vec = [&](int k) {
    const EwOperand& o = P.inputs[k];
    return (o.dtype == BG_F16 || o.dtype == BG_BF16) && ps.in_off_bytes[k] % 8 == 0;
  };
  auto term_kind = [&](int k) -> int {
    const EwOperand& o = P.inputs[k];
    if (!wide && half_vec(k)) return o.mode == A_CONTIG ? 1 : 0;     // a dense 16-bit term of an fp32 sum, widened exactly
    if (!float_vec(k) || (!wide && o.dtype != BG_F32)) return 0;
    if (o.mode == A_CONTIG) return 1;
    if (o.mode == A_STRIDED && P.ndim == 2 && P.shape[1] == P.cols && o.stride[0] == 0 && o.stride[1] == 1) return 2;
    return 0;
  };
  std::map<int, std::vector<int>> reg;   // register -> operands whose left-to-right sum it holds
  int sum_out = -1;
  auto source = [&](uint8_t r, std::vector<int>& out) -> bool {
    if ((r & kEwConst) == kEwConst) return false;
    if (r & kEwDirect) { out.assign(1, r & 0x3f); return true; }
    auto it = reg.find(r);
    if (it == reg.end()) return false;
    out = it->second;
    return true;
  };
  for (int i = 0; i < P.n_instr; ++i) {
    const EwInstr& I = P.instr[i];
    std::vector<int> a, b;
    if (I.op == E_LOAD) {
      reg[I.dst] = {(int)I.aux};
    } else if (I.op == E_COPY && (I.dst & kEwDirect)) {
      // the fp32 row sum written out as it is
      const int o = I.dst & 0x3f;
      if (I.a != (uint8_t)P.tail_reg || sum_out >= 0 || P.outputs[o].dtype != sum_dtype) return false;
      sum_out = o;
    } else if (I.op == E_COPY) {
      if (!source(I.a, a) || a.size() != 1) return false;
      reg[I.dst] = a;
    } else if (I.op == E_CVT) {
      // widening a loaded fp32 operand before it joins an fp64 sum
      if (I.type != T_F64 || !source(I.a, a) || a.size() != 1 || P.inputs[a[0]].dtype != BG_F32) return false;
      reg[I.dst] = a;
    } else if (I.op == E_ADD) {
      if (I.type != P.tail_type || !source(I.a, a) || !source(I.b, b)) return false;
      // (sum) + x and x + (sum) give the same bits; (sum) + (sum) would re-associate
      if (b.size() != 1 && a.size() != 1) return false;
      std::vector<int> v = b.size() == 1 ? a : b;
      v.push_back(b.size() == 1 ? b[0] : a[0]);
      if (v.size() > 4) return false;
      if (I.dst & kEwDirect) return false;
      reg[I.dst] = v;
    } else if (I.op == E_STORE) {
      if (I.a != (uint8_t)P.tail_reg || sum_out >= 0 || P.outputs[I.aux].dtype != sum_dtype) return false;
      sum_out = I.aux;
    } else {
      return false;
    }
  }
  auto it = reg.find(P.tail_reg);
  if (it == reg.end()) return false;
  if ((sum_out >= 0) != (P.n_outputs == 2) || sum_out == P.tail_out) return false;
  const std::vector<int>& terms = it->second;
  // a lone operand of another width than the row's stays on the interpreter
  if (terms.size() == 1 && P.inputs[terms[0]].dtype != sum_dtype) return false;
  for (size_t k = 0; k < terms.size(); ++k) {
    const int kind = term_kind(terms[k]);
    if (kind == 0 || terms[k] == P.tail_w || terms[k] == P.tail_b) return false;
    ps.ln_term[k] = terms[k];
    ps.ln_rowvec[k] = kind == 2;
  }
  ps.ln_terms = (int)terms.size();
  ps.ln_sum_out = sum_out;
  return true;
}

static int run_static_ln(Run& r, const ProgramSpec& ps) {
  const EwProgram& P = ps.prog;
  auto in_ptr = [&](int k) { return reinterpret_cast<const char*>(r.ptr[ps.in_slot[k]]) + ps.in_off_bytes[k]; };
  LnArgs a{};
  a.n_terms = ps.ln_terms;
  for (int k = 0; k < ps.ln_terms; ++k) {
    a.term[k] = in_ptr(ps.ln_term[k]);
    a.term_dtype[k] = P.inputs[ps.ln_term[k]].dtype;
    a.term_rowvec[k] = ps.ln_rowvec[k];
  }
  a.wide = P.tail_type == T_F64;
  a.sum_out = ps.ln_sum_out >= 0 ? r.ptr[ps.out_slot[ps.ln_sum_out]] : nullptr;
  a.out = r.ptr[ps.out_slot[P.tail_out]];
  a.out_dtype = P.tail_out_dtype;
  a.w = in_ptr(P.tail_w);
  a.b = in_ptr(P.tail_b);
  a.w_dtype = P.inputs[P.tail_w].dtype;
  a.b_dtype = P.inputs[P.tail_b].dtype;
  a.eps = P.tail_eps;
  a.rows = P.rows;
  a.cols = P.cols;
  if (ps.ln_planes_hi >= 0) { a.planes_hi = r.ptr[ps.ln_planes_hi]; a.planes_lo = r.ptr[ps.ln_planes_lo]; }
  if (ps.ln_out16 >= 0) { a.out16 = r.ptr[ps.ln_out16]; a.out16_dtype = ps.ln_out16_dtype; }
  cudaError_t e = launch_static_ln(a, r.ctx->stream, r.ctx->sm_count);
  if (e != cudaSuccess) return cuda_fail(r.ctx, e, "layer norm kernel launch");
  return BG_OK;
}

static int run_program(Run& r, const ProgramSpec& ps) {
  if (ps.ln_terms > 0) return run_static_ln(r, ps);
  if (ps.static_pattern >= 0) {
    const EwProgram& P = ps.prog;
    StaticArgs a{};
    for (int k = 0; k < P.n_inputs && k < 4; ++k)
      a.in[k] = reinterpret_cast<const float*>(reinterpret_cast<char*>(r.ptr[ps.in_slot[k]]) + ps.in_off_bytes[k]);
    a.out = reinterpret_cast<float*>(r.ptr[ps.out_slot[0]]);
    a.rows = P.rows;
    a.cols = P.cols;
    a.numel = P.numel;
    cudaError_t e = launch_static(ps.static_pattern, ps.static_kind, a, ps.static_arg, r.ctx->stream, r.ctx->sm_count);
    if (e != cudaSuccess) return cuda_fail(r.ctx, e, "pattern kernel launch");
    return BG_OK;
  }
  EwProgram p = ps.prog;
  for (int k = 0; k < p.n_inputs; ++k)
    p.inputs[k].ptr = reinterpret_cast<char*>(r.ptr[ps.in_slot[k]]) + ps.in_off_bytes[k];
  for (int k = 0; k < p.n_outputs; ++k) p.outputs[k].ptr = r.ptr[ps.out_slot[k]];
  cudaError_t e = ps.row ? launch_rowwise(p, r.ctx->stream, r.ctx->sm_count, r.ctx->d_status)
                         : launch_elementwise(p, r.ctx->stream, r.ctx->sm_count);
  if (e != cudaSuccess) return cuda_fail(r.ctx, e, ps.row ? "row kernel launch" : "elementwise kernel launch");
  return BG_OK;
}

void Compiler::emit_group(const std::vector<int>& members, int tail_node, int key) {
  auto ps = std::make_shared<ProgramSpec>();
  PUnit pu;
  std::string why;
  if (!build_program(members, tail_node, *ps, pu.dep_nodes, pu.out_nodes, why)) throw CompileError{-1, why};
  pu.order_key = key;
  if (ctx_->static_patterns) {
    int kind = 0, arg = 0, nin = 0;
    ps->signature = program_signature(ps->prog, &kind, &arg);
    const int pat = ps->signature.empty() ? -1 : static_pattern_id(ps->signature, &nin);
    if (pat >= 0 && nin == ps->prog.n_inputs &&
        static_shape_ok(kind, ps->prog.rows, ps->prog.cols, ps->prog.numel, ctx_->sm_count)) {
      ps->static_pattern = pat;
      ps->static_kind = kind;
      ps->static_arg = arg;
    }
    if (ps->static_pattern < 0) match_static_ln(*ps);
    if (ps->ln_terms > 0 && tail_node >= 0 && ps->prog.cols % 8 == 0 && feeds_only_split_gemms(tail_node)) {
      const int64_t n = ps->prog.rows * ps->prog.cols;
      ps->ln_planes_hi = new_slot(n * 4, false, -1);
      ps->ln_planes_lo = new_slot(n * 4, false, -1);
      pu.u.writes.push_back(ps->ln_planes_hi); pu.u.writes.push_back(ps->ln_planes_lo);
      publish_planes(tail_node, ps->ln_planes_hi, ps->ln_planes_lo, (int)punits_.size());
    }
    int dt16 = 0;
    if (ps->ln_terms > 0 && tail_node >= 0 && ps->ln_planes_hi < 0 && feeds_only_convert16(tail_node, &dt16)) {
      const int64_t n = ps->prog.rows * ps->prog.cols;
      ps->ln_out16 = new_slot(n * 2, false, -1);
      ps->ln_out16_dtype = dt16;
      pu.u.writes.push_back(ps->ln_out16);
      conv_memo_[std::make_tuple(view_[tail_node].slot, (int64_t)0, n, dt16)] = {ps->ln_out16, (int)punits_.size()};
    }
  }
  std::ostringstream nm;
  if (ps->static_pattern >= 0 || ps->ln_terms > 0) nm << "static_";
  nm << (tail_node >= 0 ? "row" : "ew") << "[";
  for (size_t i = 0; i < members.size() && i < 6; ++i) nm << (i ? "," : "") << op_name(nodes_[members[i]].op);
  if (members.size() > 6) nm << ",+" << members.size() - 6;
  if (tail_node >= 0) nm << (members.empty() ? "" : "|") << op_name(nodes_[tail_node].op);
  nm << "]";
  if (ps->ln_planes_hi >= 0) nm << "+split";
  if (ps->ln_out16 >= 0) nm << "+cast16";
  pu.u.name = nm.str();
  pu.u.fn = [ps](Run& r) { return run_program(r, *ps); };
  add_unit(std::move(pu));
}

void Compiler::emit_row_standalone(int r, int key) {
  std::vector<int> none;
  emit_group(none, r, key);
}

void Compiler::emit_const_fill(int n, int key) {
  // a constant that must exist in memory: CONST -> STORE over the node's shape
  auto ps = std::make_shared<ProgramSpec>();
  EwProgram& P = ps->prog;
  memset(&P, 0, sizeof(P));
  const View v = view_[n];
  EwType c = cls_of(v.dtype);
  int64_t bits;
  if (c == T_F32 || c == T_F64) { double d = v.cf; memcpy(&bits, &d, 8); } else bits = v.ci;
  P.consts[0] = bits;
  P.n_consts = 1;
  P.instr[0] = {E_CONST, (uint8_t)c, 0, 0, 0, 0, 0};
  P.instr[1] = {E_STORE, (uint8_t)c, 0, 0, 0, 0, 0};
  P.n_instr = 2;
  P.n_regs = 1;
  P.wide = (c == T_F64 || c == T_I64);
  P.ndim = 1;
  P.numel = nodes_[n].numel();
  P.shape[0] = P.numel;
  P.n_outputs = 1;
  P.outputs[0].dtype = v.dtype;
  P.outputs[0].vec_ok = 1;
  View nv;
  nv.set_dense(nodes_[n].shape, nodes_[n].rank);
  nv.dtype = v.dtype;
  nv.slot = new_slot(P.numel * dtype_size(v.dtype), false, n);
  view_[n] = nv;
  ps->out_slot[0] = nv.slot;
  PUnit pu;
  pu.order_key = key;
  pu.out_nodes = {n};
  pu.u.name = "fill[CONST]";
  pu.u.fn = [ps](Run& r) { return run_program(r, *ps); };
  add_unit(std::move(pu));
}

void Compiler::emit_copy(int n, const View& sv, int src, int key) {
  // dense copy of a strided view (RESHAPE of a permuted tensor, or a view that is the plan root)
  // into the slot already assigned to node n
  const int es = dtype_size(nodes_[n].dtype);
  const int64_t numel = nodes_[n].numel();
  const int in_slot = sv.slot, out_slot = view_[n].slot;
  StridedView tmpl{};
  tmpl.dtype = sv.dtype;
  tmpl.rank = sv.rank;
  for (int d = 0; d < sv.rank; ++d) { tmpl.shape[d] = sv.shape[d]; tmpl.stride[d] = sv.stride[d]; }
  const int64_t off_bytes = sv.off * es;
  PUnit pu;
  pu.order_key = key;
  pu.dep_nodes = {src};
  pu.out_nodes = {n};
  pu.u.name = "copy[strided]";
  pu.u.fn = [=](Run& r) {
    StridedView v = tmpl;
    v.ptr = reinterpret_cast<char*>(r.ptr[in_slot]) + off_bytes;
    cudaError_t e = launch_strided_copy(v, r.ptr[out_slot], numel, r.ctx->stream);
    return e == cudaSuccess ? (int)BG_OK : cuda_fail(r.ctx, e, "strided copy launch");
  };
  add_unit(std::move(pu));
}

void Compiler::emit_generic_reduce(int n, int key) {
  // REDUCE over a contiguous block of non-trailing axes of a dense tensor: [outer, R, inner]
  const Node& t = nodes_[n];
  const int x = resolve(t.in[0]);
  const View xv = view_[x];
  const Node& xn = nodes_[x];
  const uint64_t mask = (uint64_t)t.iarg[1];
  int lo = -1, hi = -1;
  for (int d = 0; d < xn.rank; ++d)
    if ((mask >> d) & 1) { if (lo < 0) lo = d; hi = d; }
  int64_t outer = 1, R = 1, inner = 1;
  for (int d = 0; d < xn.rank; ++d) {
    if (d < lo) outer *= xn.shape[d]; else if (d <= hi) R *= xn.shape[d]; else inner *= xn.shape[d];
  }
  if (t.iarg[0] < 0 || t.iarg[0] > BG_RED_PROD) err(BG_ERR_INVALID, "REDUCE: unknown reduction");
  if (t.iarg[0] == BG_RED_PROD && xv.dtype != BG_F32 && xv.dtype != BG_F64 && xv.dtype != BG_I64)
    err(BG_ERR_UNSUPPORTED, "REDUCE prod: float32, float64 and int64 only");
  own_slot(n);
  const int in_slot = xv.slot, out_slot = view_[n].slot, in_dt = xv.dtype, out_dt = t.dtype, rop = (int)t.iarg[0];
  const int64_t off_bytes = xv.off * dtype_size(xv.dtype);
  PUnit pu;
  pu.order_key = key;
  pu.dep_nodes = {x};
  pu.out_nodes = {n};
  pu.u.name = "reduce[strided-axis]";
  pu.u.fn = [=](Run& r) {
    cudaError_t e = launch_reduce_generic(reinterpret_cast<char*>(r.ptr[in_slot]) + off_bytes, r.ptr[out_slot], in_dt, out_dt,
                                          rop, outer, R, inner, r.ctx->stream);
    return e == cudaSuccess ? (int)BG_OK : cuda_fail(r.ctx, e, "reduce launch");
  };
  add_unit(std::move(pu));
}

void Compiler::emit_generic_softmax(int n, int key) {
  const Node& t = nodes_[n];
  const int x = resolve(t.in[0]);
  const View xv = view_[x];
  const Node& xn = nodes_[x];
  if (t.dtype != BG_F32 && t.dtype != BG_F64) err(BG_ERR_UNSUPPORTED, "FUSED_SOFTMAX: float32/float64 only");
  if (xv.dtype != t.dtype) err(BG_ERR_UNSUPPORTED, "FUSED_SOFTMAX: input dtype differs from output dtype");
  const int axis = (int)t.iarg[0];
  int64_t outer = 1, R = xn.shape[axis], inner = 1;
  for (int d = 0; d < axis; ++d) outer *= xn.shape[d];
  for (int d = axis + 1; d < xn.rank; ++d) inner *= xn.shape[d];
  own_slot(n);
  const int in_slot = xv.slot, out_slot = view_[n].slot, dt = t.dtype;
  const int64_t off_bytes = xv.off * dtype_size(xv.dtype);
  PUnit pu;
  pu.order_key = key;
  pu.dep_nodes = {x};
  pu.out_nodes = {n};
  pu.u.name = "softmax[strided-axis]";
  pu.u.fn = [=](Run& r) {
    cudaError_t e = launch_softmax_generic(reinterpret_cast<char*>(r.ptr[in_slot]) + off_bytes, r.ptr[out_slot], dt, outer, R,
                                           inner, r.ctx->stream);
    return e == cudaSuccess ? (int)BG_OK : cuda_fail(r.ctx, e, "softmax launch");
  };
  add_unit(std::move(pu));
}


// Which tensor-core encoding a MATMUL node can use, judged from the operand views alone.
int Compiler::tc_mode(int n) {
  const Node& t = nodes_[n];
  if (!ctx_->tensor_cores || t.in.size() != 2) return -1;
  const View& av = view_[resolve(t.in[0])];
  const View& bv = view_[resolve(t.in[1])];
  if (av.is_const || bv.is_const || av.rank != 2 || bv.rank != 2 || t.rank != 2) return -1;
  const int64_t M = av.shape[0], K = av.shape[1], N = bv.shape[1];
  if (bv.shape[0] != K || M * N * K < (1ll << 24)) return -1;
  int mode = -1;
  if (av.dtype == bv.dtype && (av.dtype == BG_F16 || av.dtype == BG_BF16) && t.dtype == av.dtype) mode = 0;
  else if (av.dtype == BG_F32 && bv.dtype == BG_F32 && t.dtype == BG_F32) mode = 1;
  else if (t.dtype == BG_F64 && (av.dtype == BG_F32 || av.dtype == BG_F64) && (bv.dtype == BG_F32 || bv.dtype == BG_F64) &&
           (ctx_->f64_mode == 1 || (ctx_->f64_mode == 2 && !has_f64_leaf_))) mode = 1;
  if (mode < 0) return -1;
  if (!tc_gemm_supported(M, N, K, mode == 0 ? av.dtype : BG_F32)) return -1;
  return mode;
}

// act_expr() of the reference's tanh GELU of x: 0.5 x (1 + tanh(k (x + 0.044715 x^3))) with tanh written out in exponentials.
static std::string gelu_expr_text() {
  const std::string Z = "mul(c0.797885,add(x,mul(mul(mul(c0.044715,x),x),x)))";
  return "mul(mul(c0.5,x),add(c1,div(add(exp(" + Z + "),neg(exp(neg(" + Z + ")))),add(exp(" + Z + "),exp(neg(" + Z + "))))))";
}

// The nodes that read the storage of f: its consumers, followed through the views that alias it.  False when the
// storage has to hold f as the graph types it -- f (or a view of it) is the plan's root, f is not a dense buffer of
// its own, or a reshape of it became a copy.
bool Compiler::storage_readers(int f, std::vector<int>& readers) {
  if (!ctx_->fusion || !ctx_->static_patterns || f == root_) return false;
  const View& fv = view_[f];
  if (fv.is_const || fv.off != 0 || !fv.contiguous()) return false;
  std::vector<int> stack{f};
  std::set<int> seen;
  while (!stack.empty()) {
    const int v = stack.back();
    stack.pop_back();
    if (!seen.insert(v).second) continue;
    if (v == root_) return false;
    for (int c : cons_[v]) {
      if (kind_[c] == K_DEAD) continue;
      if (kind_[c] == K_VIEW || kind_[c] == K_ALIAS) {
        if (view_[c].slot != fv.slot) return false;
        stack.push_back(c);
      } else {
        readers.push_back(c);
      }
    }
  }
  return true;
}

// True when the value of node f is read by nothing but tensor-core split products that take all of it as their dense
// [M, K] A operand (through reshapes), K a multiple of 8: the unit that computes f can then store the operand planes
// of those products (tf32(x); bf16(x); bf16(x - tf32(x))) in place of f itself, and no pass of its own splits f.
bool Compiler::feeds_only_split_gemms(int f) {
  std::vector<int> readers;
  const View& fv = view_[f];
  if ((fv.dtype != BG_F32 && fv.dtype != BG_F64) || !storage_readers(f, readers)) return false;
  const int64_t numel = fv.numel();
  for (int c : readers) {
    const Node& m = nodes_[c];
    if (m.op != BG_OP_MATMUL || kind_[c] != K_OTHER || attn_plan_.count(c) || attn_absorbed_.count(c) || tc_mode(c) != 1) return false;
    const View& av = view_[resolve(m.in[0])];
    const View& bv = view_[resolve(m.in[1])];
    if (av.slot != fv.slot || bv.slot == fv.slot) return false;
    if (av.off != 0 || av.rank != 2 || av.stride[1] != 1 || av.stride[0] != av.shape[1] || av.shape[0] * av.shape[1] != numel ||
        av.shape[1] % 8 != 0)
      return false;
  }
  return !readers.empty();
}

// True when the fp32 / fp64 value of node f is read by nothing but CASTs to one 16-bit type that tensor-core GEMMs
// absorbed as the conversion of their dense A operand (autocast Linears after a LayerNorm): the unit that computes f
// can then store the 16-bit rows itself, registered where those GEMMs look for an activation already converted.
bool Compiler::feeds_only_convert16(int f, int* dtype16) {
  std::vector<int> readers;
  const View& fv = view_[f];
  if ((fv.dtype != BG_F32 && fv.dtype != BG_F64) || !storage_readers(f, readers)) return false;
  const int64_t numel = fv.numel();
  // the casts that GEMMs of this plan absorbed as conversions of all of f
  std::set<int> a_casts;
  int dt = -1;
  for (const auto& kv : gemm_cast_src_) {
    const int n = kv.first, sa = kv.second.first;
    if (sa < 0 || view_[sa].slot != fv.slot) continue;
    const int a = resolve(nodes_[n].in[0]);
    const View& av = view_[a];
    int ca = -1;
    if (absorbable_cast(a, av.dtype, ca, true) != sa || ca < 0) return false;
    if (view_[sa].off + av.off != 0 || av.rank != 2 || av.shape[0] * av.shape[1] != numel || numel % 8 != 0) return false;
    if (dt >= 0 && dt != av.dtype) return false;
    dt = av.dtype;
    a_casts.insert(ca);
  }
  if (a_casts.empty()) return false;
  for (int c : readers)
    if (!a_casts.count(c)) return false;
  *dtype16 = dt;
  return true;
}

// True when the fp64 value of node f -- the result of a 3xTF32 product, so every element is an fp32 number -- is read
// by nothing but fused 3xTF32 attentions (as Q, K or V, through views).  Those kernels compute on fp32: the product
// then stores fp32 into f's storage and the attention reads fp32 rows, half the bytes on either side and no pass
// that narrows Q and K.
bool Compiler::feeds_only_attention32(int f) {
  std::vector<int> readers;
  if (view_[f].dtype != BG_F64 || !storage_readers(f, readers)) return false;
  const View& fv = view_[f];
  for (int c : readers) {
    // the Q K^T product inside a fused attention, or its final product (absorbed casts of other kernels are not)
    const bool inner_product = attn_absorbed_.count(c) && nodes_[c].op == BG_OP_MATMUL;
    if (!attn_plan_.count(c) && !inner_product) return false;
  }
  bool any = false;
  for (const auto& kv : attn_plan_) {
    const AttnPlan& ap = kv.second;
    const int ops[3] = {ap.q, ap.kt, ap.v};
    const int srcs[3] = {ap.q_src, ap.kt_src, ap.v_src};
    for (int i = 0; i < 3; ++i) {
      if (view_[ops[i]].slot != fv.slot) continue;
      if (ap.mode != 1 || srcs[i] >= 0) return false;
      any = true;
    }
    if (ap.mask >= 0 && view_[ap.mask].slot == fv.slot) return false;
    if (ap.scale_node >= 0 && view_[ap.scale_node].slot == fv.slot) return false;
  }
  return any;
}

bool Compiler::narrow_store(int n) {
  auto final_of = [&](int m) {
    auto it = epi_plan_.find(m);
    return it != epi_plan_.end() ? it->second.final_node : m;
  };
  auto one = [&](int m) {
    auto it = epi_plan_.find(m);
    if (it != epi_plan_.end() && it->second.act != TC_ACT_NONE) return false;
    return tc_mode(m) == 1 && nodes_[final_of(m)].dtype == BG_F64 && feeds_only_attention32(final_of(m));
  };
  auto gi = gemm_group_of_.find(n);
  if (gi == gemm_group_of_.end()) return one(n);
  for (int m : gemm_groups_[gi->second].members)     // one store type per joint launch
    if (!one(m)) return false;
  return true;
}

// The unit `punit` (being built: the next one added) stores the planes of f: the products that read f find them
// where they would have looked for a split made by an earlier product of the plan.
void Compiler::publish_planes(int f, int hi, int lo, int punit) {
  split_memo_[std::make_tuple(view_[f].slot, (int64_t)0, view_[f].numel())] = {hi, lo, punit};
}

// A small 2-D fp32 MATMUL (below the tensor-core threshold) runs on the split-K kernel of gemm_simt.cu.
bool Compiler::small_gemm(int n, int* splits, int64_t* partial_bytes) {
  const Node& t = nodes_[n];
  if (!ctx_->fusion || t.in.size() != 2 || t.rank != 2 || t.dtype != BG_F32 || tc_mode(n) >= 0) return false;
  const View& av = view_[resolve(t.in[0])];
  const View& bv = view_[resolve(t.in[1])];
  if (av.is_const || bv.is_const || av.rank != 2 || bv.rank != 2 || av.dtype != BG_F32 || bv.dtype != BG_F32) return false;
  GemmProblem gp{};
  gp.m = av.shape[0];
  gp.k = av.shape[1];
  gp.n = bv.shape[1];
  if (bv.shape[0] != gp.k) return false;
  gp.a.dtype = gp.b.dtype = gp.c_dtype = BG_F32;
  return gemm_small_plan(gp, ctx_->sm_count, splits, partial_bytes);
}

// Expression of `node` in terms of the value `x`, constants, and elementwise members of group g.
std::string Compiler::act_expr(int node, int x, int g, int depth) {
  node = resolve(node);
  if (node == x) return "x";
  if (depth > 64) return "?";
  const Node& n = nodes_[node];
  if (kind_[node] == K_CONST) {
    char buf[64];
    snprintf(buf, sizeof(buf), "c%.6g", view_[node].is_const ? (dtype_is_float(n.dtype) ? view_[node].cf : (double)view_[node].ci) : 0.0);
    return buf;
  }
  if (kind_[node] != K_EW || find(node) != g) return "?";
  std::string nm;
  switch (n.op) {
    case BG_OP_ADD: nm = "add"; break;
    case BG_OP_MUL: nm = "mul"; break;
    case BG_OP_DIV: nm = "div"; break;
    case BG_OP_NEG: nm = "neg"; break;
    case BG_OP_EXP: nm = "exp"; break;
    case BG_OP_WHERE: nm = "where"; break;
    case BG_OP_CMP: nm = std::string("cmp") + std::to_string((int)n.iarg[0]); break;
    default: return "?";
  }
  std::string out = nm + "(";
  for (size_t i = 0; i < n.in.size(); ++i) out += (i ? "," : "") + act_expr(n.in[i], x, g, depth + 1);
  return out + ")";
}

// Fold the elementwise group that consumes a tensor-core product into the GEMM's epilogue when the
// whole group is [CAST to fp32] -> [+ bias row] -> [relu | gelu] of that product.
// The fp32 node whose CAST to `dtype16` is all that stands between it and `node` (through views only), when that
// cast exists for this one consumer chain, is an elementwise group of its own and reads a dense fp32 tensor; -1 else.
int Compiler::absorbable_cast(int node, int dtype16, int& cast_node, bool allow_f64) {
  auto single = [&](int v) {
    std::set<int> c(cons_[v].begin(), cons_[v].end());
    return c.size() == 1 && v != root_;
  };
  int pnode = node;
  while (kind_[pnode] == K_VIEW || kind_[pnode] == K_ALIAS) {
    if (!single(pnode)) return -1;
    pnode = resolve(nodes_[pnode].in[0]);
  }
  if (kind_[pnode] != K_EW || nodes_[pnode].op != BG_OP_CAST || nodes_[pnode].dtype != dtype16 || !single(pnode)) return -1;
  const int g = find(pnode);
  for (int i = 0; i < (int)nodes_.size(); ++i)
    if (i != pnode && kind_[i] == K_EW && find(i) == g) return -1;    // fused with other elementwise work
  const int src = resolve(nodes_[pnode].in[0]);
  const View& sv = view_[src];
  if (sv.is_const || sv.slot < 0 || !(sv.dtype == BG_F32 || (allow_f64 && sv.dtype == BG_F64)) || !sv.contiguous() ||
      sv.rank != nodes_[pnode].rank)
    return -1;
  for (int d = 0; d < sv.rank; ++d)
    if (sv.shape[d] != nodes_[pnode].shape[d]) return -1;
  cast_node = pnode;
  return src;
}

// Autocast Linear layers reach the tensor-core GEMM as MATMUL(CAST(x), PERMUTE(CAST(W))).  Where such a cast only
// feeds this GEMM, the GEMM unit converts the operand itself with a vectorised pass (and keeps the converted copy
// of a weight bound by handle with that handle), so the interpreter's CAST kernels and their outputs disappear.
void Compiler::plan_gemm_groups() {
  gemm_groups_.clear();
  gemm_group_of_.clear();
  if (!ctx_->fusion || !ctx_->tensor_cores || !ctx_->gemm_groups) return;
  typedef std::vector<int64_t> Key;
  std::map<Key, std::vector<int>> buckets;
  for (int n = 0; n < (int)nodes_.size(); ++n) {
    if (kind_[n] != K_OTHER || nodes_[n].op != BG_OP_MATMUL || nodes_[n].rank != 2) continue;
    if (attn_plan_.count(n) || attn_absorbed_.count(n)) continue;
    const int mode = tc_mode(n);
    if (mode < 0) continue;
    const int a = resolve(nodes_[n].in[0]), b = resolve(nodes_[n].in[1]);
    const View& av = view_[a];
    const View& bv = view_[b];
    int a_f32 = -1, b_f32 = -1;
    {
      auto cs = gemm_cast_src_.find(n);
      if (cs != gemm_cast_src_.end()) { a_f32 = cs->second.first; b_f32 = cs->second.second; }
    }
    // B (or the fp32 tensor behind its absorbed cast) is bound from outside: nothing of this plan produces it
    const int b_leaf = b_f32 >= 0 ? b_f32 : b;
    if (!leaflike_[b_leaf] || bv.is_const || view_[b_leaf].slot < 0 || !cp_->slots[view_[b_leaf].slot].external) continue;
    const int64_t M = av.shape[0], K = av.shape[1], N = bv.shape[1];
    if (M <= 128 || N <= 128) continue;                       // the joint launch is a CTA-pair launch
    if (!(bv.stride[0] == 1 && bv.stride[1] == K)) continue;  // B read in place
    int fin = n, bias_dt = -1, act = 0, round_acc = 0, wide = 0;
    auto ep = epi_plan_.find(n);
    if (ep != epi_plan_.end()) {
      fin = ep->second.final_node; act = ep->second.act; round_acc = ep->second.round_acc; wide = ep->second.wide;
      if (ep->second.bias_node >= 0) {
        if (!leaflike_[ep->second.bias_node]) continue;
        bias_dt = view_[ep->second.bias_node].dtype;
      }
    }
    Key key = {a_f32 >= 0 ? a_f32 : a, M, N, K, mode, av.dtype, bv.dtype, nodes_[n].dtype, nodes_[fin].dtype, act, round_acc, wide, bias_dt,
               a_f32, b_f32 >= 0 ? 1 : 0};
    buckets[key].push_back(n);
  }
  for (auto& kv : buckets) {
    const std::vector<int>& mem = kv.second;
    for (size_t i = 0; i + 1 < mem.size(); i += 3) {
      GemmGroup g;
      for (size_t j = i; j < mem.size() && j < i + 3; ++j) g.members.push_back(mem[j]);
      g.run = std::make_shared<GroupRun>();
      for (int m : g.members) gemm_group_of_[m] = (int)gemm_groups_.size();
      gemm_groups_.push_back(std::move(g));
    }
  }
}

void Compiler::plan_gemm_casts() {
  gemm_cast_src_.clear();
  if (!ctx_->fusion || !ctx_->tensor_cores) return;
  for (int n = 0; n < (int)nodes_.size(); ++n) {
    if (kind_[n] != K_OTHER || nodes_[n].op != BG_OP_MATMUL) continue;
    if (attn_plan_.count(n) || attn_absorbed_.count(n)) continue;
    if (tc_mode(n) != 0) continue;
    const int a = resolve(nodes_[n].in[0]), b = resolve(nodes_[n].in[1]);
    const View& av = view_[a];
    const View& bv = view_[b];
    const int64_t K = av.shape[1];
    // only operands the kernel reads in place: A dense [M,K], B dense [N,K] seen as [K,N]
    const bool a_dense = av.stride[1] == 1 && av.stride[0] == K;
    const bool b_kmajor = bv.stride[0] == 1 && bv.stride[1] == K;
    int ca = -1, cb = -1;
    // an activation may also be a float64 tensor (LayerNorm outputs of autocast graphs are): the conversion pass reads it
    int sa = a_dense ? absorbable_cast(a, av.dtype, ca, true) : -1;
    int sb = b_kmajor ? absorbable_cast(b, bv.dtype, cb) : -1;
    if (sa >= 0 && sb >= 0 && ca == cb) sb = -1;
    // the conversion pass moves eight elements per step: the operand must start on a 32-byte boundary of its slot
    if (sa >= 0 && (view_[sa].off + av.off) % 8 != 0) sa = -1;
    if (sb >= 0 && (view_[sb].off + bv.off) % 8 != 0) sb = -1;
    if (sa < 0 && sb < 0) continue;
    gemm_cast_src_[n] = {sa, sb};
    if (sa >= 0) attn_absorbed_.insert(ca);
    if (sb >= 0) attn_absorbed_.insert(cb);
  }
}

void Compiler::plan_tc_epilogues(const std::map<int, std::vector<int>>& groups) {
  epi_plan_.clear();
  absorbed_groups_.clear();
  if (!ctx_->fusion) return;
  const std::string gelu = gelu_expr_text();
  const std::string relu = "where(cmp" + std::to_string((int)BG_CMP_GT) + "(x,c0),x,c0)";
  for (int n = 0; n < (int)nodes_.size(); ++n) {
    if (kind_[n] != K_OTHER || nodes_[n].op != BG_OP_MATMUL) continue;
    if (attn_plan_.count(n) || attn_absorbed_.count(n)) continue;
    int small_splits = 0;
    int64_t small_bytes = 0;
    const bool small = tc_mode(n) < 0 && small_gemm(n, &small_splits, &small_bytes);   // fp32 bias row and ReLU only
    if (tc_mode(n) < 0 && !small) continue;
    const int64_t N = nodes_[n].shape[1];
    EpiPlan ep;
    std::set<int> absorbed;
    int cur = n;
    auto sole_consumer = [&](int v) -> int {
      std::set<int> c(cons_[v].begin(), cons_[v].end());
      return c.size() == 1 && v != root_ ? *c.begin() : -1;
    };
    int nx = sole_consumer(cur);
    if (nx < 0 || kind_[nx] != K_EW) continue;
    const int g = find(nx);
    if (tail_of_group_[g] >= 0) continue;
    // optional CAST of a 16-bit product to fp32
    if (nodes_[nx].op == BG_OP_CAST && nodes_[nx].dtype == BG_F32 && (nodes_[n].dtype == BG_F16 || nodes_[n].dtype == BG_BF16)) {
      ep.round_acc = nodes_[n].dtype + 1;
      absorbed.insert(nx);
      cur = nx;
      nx = sole_consumer(cur);
    } else if (nodes_[n].dtype == BG_F16 || nodes_[n].dtype == BG_BF16) {
      continue;   // a 16-bit result is stored as is
    }
    // optional bias row
    if (nx >= 0 && kind_[nx] == K_EW && find(nx) == g && nodes_[nx].op == BG_OP_ADD && nodes_[nx].in.size() == 2) {
      const int i0 = resolve(nodes_[nx].in[0]), i1 = resolve(nodes_[nx].in[1]);
      const int other = i0 == cur ? i1 : (i1 == cur ? i0 : -1);
      if (other >= 0 && other != cur) {
        const View& bv = view_[other];
        const bool row = !bv.is_const && bv.numel() == N && bv.contiguous() && bv.rank >= 1 && bv.shape[bv.rank - 1] == N &&
                         leaflike_[other] && (bv.dtype == BG_F32 || bv.dtype == BG_F64 || bv.dtype == BG_F16);
        if (row && (nodes_[nx].dtype == BG_F32 || nodes_[nx].dtype == BG_F64) &&
            (!small || (bv.dtype == BG_F32 && nodes_[nx].dtype == BG_F32))) {
          ep.bias_node = other;
          absorbed.insert(nx);
          cur = nx;
        }
      }
    }
    if (cur == n) continue;   // nothing linear to fold
    // activation: the rest of the group must be exactly relu(x) or gelu(x) of the folded value
    const std::vector<int>& mem = groups.at(g);
    std::vector<int> mats;
    for (int m : mem)
      if (need_mat_[m]) mats.push_back(m);
    int final_node = -1;
    bool out16 = false;       // the group ends in the CAST back to the product's 16-bit type: the epilogue stores that type
    if (mats.size() == 1) {
      int target = mats[0];
      const Node& mn = nodes_[target];
      if (!small && ep.round_acc && mn.op == BG_OP_CAST && mn.in.size() == 1 && mn.dtype == nodes_[n].dtype) {
        const int inner = resolve(mn.in[0]);
        if (kind_[inner] == K_EW && find(inner) == g && nodes_[inner].dtype == BG_F32) { target = inner; out16 = true; }
      }
      if (target == cur) final_node = mats[0];
      else {
        const std::string e = act_expr(target, cur, g, 0);
        if (e == relu) { ep.act = TC_ACT_RELU; final_node = mats[0]; }
        else if (e == gelu) { ep.act = TC_ACT_GELU; final_node = mats[0]; }
      }
    }
    if (final_node < 0) continue;
    // every member of the group must be part of what was folded
    bool all = true;
    for (int m : mem) {
      if (absorbed.count(m) || m == final_node) continue;
      if (ep.act == TC_ACT_NONE) { all = false; break; }
      // activation interior nodes are reachable only from final_node; accept members that feed it
    }
    if (!all) continue;
    if (ep.act != TC_ACT_NONE) {
      // interior check: each member must be reachable from final_node within the group
      std::set<int> reach;
      std::vector<int> stack{final_node};
      while (!stack.empty()) {
        int v = stack.back();
        stack.pop_back();
        if (!reach.insert(v).second) continue;
        for (int in : nodes_[v].in) {
          int r = resolve(in);
          if (kind_[r] == K_EW && find(r) == g) stack.push_back(r);
        }
      }
      for (int m : mem)
        if (!reach.count(m)) { all = false; break; }
      if (!all) continue;
    }
    const int fdt = nodes_[final_node].dtype;
    if (fdt != BG_F32 && fdt != BG_F64 && !out16) continue;
    if (small && (fdt != BG_F32 || ep.act == TC_ACT_GELU)) continue;
    ep.wide = out16 ? 0 : fdt == BG_F64 && ep.act == TC_ACT_GELU && nodes_[cur].dtype != BG_F64 ? 1 : (fdt == BG_F64 ? 1 : 0);
    ep.final_node = final_node;
    ep.group = g;
    epi_plan_[n] = ep;
    absorbed_groups_.insert(g);
  }
}

// Recognise softmax(scale * Q K^T [+ mask]) V as built by scaled_dot_product_attention
// (packages/browsergrad-jit/src/python/_functional.py:1505-1534) or by the typed attention op:
//   MATMUL(q, permuted k) -> [CAST] -> MUL(scale) -> [ADD(mask) | WHERE(mask, -inf, .)] -> FUSED_SOFTMAX -> [CAST] -> MATMUL(., v)
// Every interior value must have that single consumer.
bool Compiler::match_attention(int n, AttnPlan& ap, std::vector<int>& interior) {
  const Node& fin = nodes_[n];
  if (fin.op != BG_OP_MATMUL || fin.rank != 4 || fin.in.size() != 2) return false;
  auto single = [&](int v) {
    std::set<int> c(cons_[v].begin(), cons_[v].end());
    return c.size() == 1 && v != root_;
  };
  int cur = resolve(fin.in[0]);
  ap.v = resolve(fin.in[1]);
  if (!single(cur)) return false;
  if (nodes_[cur].op == BG_OP_CAST) { interior.push_back(cur); cur = resolve(nodes_[cur].in[0]); if (!single(cur)) return false; }
  if (nodes_[cur].op != BG_OP_FUSED_SOFTMAX || nodes_[cur].rank != 4 || nodes_[cur].iarg[0] != 3) return false;
  interior.push_back(cur);
  cur = resolve(nodes_[cur].in[0]);
  if (!single(cur)) return false;
  const int64_t B = fin.shape[0], H = fin.shape[1], Sq = fin.shape[2], D = fin.shape[3];
  const int64_t Sk = nodes_[cur].shape[3];
  auto is_scores = [&](int v) {
    const Node& x = nodes_[v];
    return x.rank == 4 && x.shape[0] == B && x.shape[1] == H && x.shape[2] == Sq && x.shape[3] == Sk;
  };
  if (!is_scores(cur)) return false;
  // mask
  if (nodes_[cur].op == BG_OP_ADD && nodes_[cur].in.size() == 2) {
    const int a = resolve(nodes_[cur].in[0]), b = resolve(nodes_[cur].in[1]);
    int m = -1, nx = -1;
    for (int k = 0; k < 2; ++k) {
      const int cand = k ? b : a, other = k ? a : b;
      const View& mv = view_[cand];
      if (leaflike_[cand] && !mv.is_const && mv.dtype == BG_F32 && mv.rank >= 2 && mv.rank <= 4 && mv.shape[mv.rank - 1] == Sk &&
          mv.shape[mv.rank - 2] == Sq && mv.stride[mv.rank - 1] == 1 && mv.stride[mv.rank - 2] == Sk && kind_[other] != K_LEAF) {
        m = cand; nx = other;
        break;
      }
    }
    if (m >= 0) {
      ap.mask = m;
      interior.push_back(cur);
      cur = nx;
      if (!single(cur) || !is_scores(cur)) return false;
    }
  } else if (nodes_[cur].op == BG_OP_WHERE && nodes_[cur].in.size() == 3) {
    const int c = resolve(nodes_[cur].in[0]), f = resolve(nodes_[cur].in[1]), x = resolve(nodes_[cur].in[2]);
    const View& mv = view_[c];
    const View& fv = view_[f];
    const bool neg_inf = fv.is_const && dtype_is_float(fv.dtype) && fv.cf < 0 && fv.cf * 2 == fv.cf;
    if (!(leaflike_[c] && !mv.is_const && mv.dtype == BG_BOOL && neg_inf && mv.rank >= 2 && mv.rank <= 4 &&
          mv.shape[mv.rank - 1] == Sk && mv.shape[mv.rank - 2] == Sq && mv.stride[mv.rank - 1] == 1 && mv.stride[mv.rank - 2] == Sk))
      return false;
    ap.mask = c;
    ap.mask_is_bool = 1;
    interior.push_back(cur);
    cur = x;
    if (!single(cur) || !is_scores(cur)) return false;
  }
  if (ap.mask >= 0) {
    const View& mv = view_[ap.mask];
    for (int d = 0; d < mv.rank - 2; ++d) {
      const int64_t want = (mv.rank - 2 - d) == 2 ? B : H;   // leading dims line up with [B, H] from the right
      if (mv.shape[d] != 1 && mv.shape[d] != want) return false;
    }
  }
  // scale
  if (nodes_[cur].op == BG_OP_MUL && nodes_[cur].in.size() == 2) {
    const int a = resolve(nodes_[cur].in[0]), b = resolve(nodes_[cur].in[1]);
    int nx = -1;
    for (int k = 0; k < 2; ++k) {
      const int cand = k ? b : a, other = k ? a : b;
      const View& sv = view_[cand];
      if (sv.is_const && dtype_is_float(sv.dtype)) { ap.scale_const = sv.cf; ap.scale_node = -1; nx = other; break; }
      if (leaflike_[cand] && sv.dtype == BG_F32 && sv.rank == 4 && sv.contiguous() && sv.shape[0] == B && sv.shape[1] == H &&
          sv.shape[2] == Sq && sv.shape[3] == Sk && kind_[other] != K_LEAF) {
        ap.scale_node = cand; nx = other; break;
      }
    }
    if (nx < 0) return false;
    interior.push_back(cur);
    cur = nx;
    if (!single(cur) || !is_scores(cur)) return false;
  }
  if (nodes_[cur].op == BG_OP_CAST) { interior.push_back(cur); cur = resolve(nodes_[cur].in[0]); if (!single(cur) || !is_scores(cur)) return false; }
  const Node& qk = nodes_[cur];
  if (qk.op != BG_OP_MATMUL || qk.in.size() != 2) return false;
  interior.push_back(cur);
  ap.q = resolve(qk.in[0]);
  ap.kt = resolve(qk.in[1]);
  const View& qv = view_[ap.q];
  const View& kv = view_[ap.kt];
  const View& vv = view_[ap.v];
  if (qv.is_const || kv.is_const || vv.is_const || qv.rank != 4 || kv.rank != 4 || vv.rank != 4) return false;
  if (qv.shape[0] != B || qv.shape[1] != H || qv.shape[2] != Sq || qv.shape[3] != D) return false;
  if (kv.shape[0] != B || kv.shape[1] != H || kv.shape[2] != D || kv.shape[3] != Sk) return false;
  if (vv.shape[0] != B || vv.shape[1] != H || vv.shape[2] != Sk || vv.shape[3] != D) return false;
  // encodings
  const int qd = qv.dtype, kd = kv.dtype, vd = vv.dtype, od = fin.dtype;
  if ((qd == BG_F16 || qd == BG_BF16) && kd == qd && vd == qd && od == qd && qk.dtype == qd) { ap.mode = 0; ap.ab_dtype = qd; }
  else if (qd == BG_F32 && kd == BG_F32 && vd == BG_F32 && od == BG_F32) { ap.mode = 1; ap.ab_dtype = BG_F32; }
  else if (od == BG_F64 && (ctx_->f64_mode == 1 || (ctx_->f64_mode == 2 && !has_f64_leaf_)) &&
           (qd == BG_F32 || qd == BG_F64) && (kd == BG_F32 || kd == BG_F64) && (vd == BG_F32 || vd == BG_F64)) { ap.mode = 1; ap.ab_dtype = BG_F32; }
  else return false;
  if (ap.mode == 0) {
    // An autocast graph feeds Q, K, V through CAST(float32 -> 16 bit) nodes.  When such a cast exists only for
    // this attention and reads a dense fp32 tensor, the operand staging pass does the rounding itself (same
    // round-to-nearest-even), so the cast's own kernel and its 16-bit copy disappear.
    auto cast_source = [&](int node, int& cast_node) -> int {
      int pnode = node;
      while (kind_[pnode] == K_VIEW || kind_[pnode] == K_ALIAS) {
        if (!single(pnode)) return -1;
        pnode = resolve(nodes_[pnode].in[0]);
      }
      if (kind_[pnode] != K_EW || nodes_[pnode].op != BG_OP_CAST || nodes_[pnode].dtype != ap.ab_dtype || !single(pnode)) return -1;
      const int g = find(pnode);
      for (int i = 0; i < (int)nodes_.size(); ++i)
        if (i != pnode && kind_[i] == K_EW && find(i) == g) return -1;    // fused with other elementwise work
      const int src = resolve(nodes_[pnode].in[0]);
      const View& sv = view_[src];
      if (sv.is_const || sv.slot < 0 || sv.dtype != BG_F32 || !sv.contiguous() || sv.rank != nodes_[pnode].rank) return -1;
      for (int d = 0; d < sv.rank; ++d)
        if (sv.shape[d] != nodes_[pnode].shape[d]) return -1;
      cast_node = pnode;
      return src;
    };
    int* srcs[3] = {&ap.q_src, &ap.kt_src, &ap.v_src};
    const int operands[3] = {ap.q, ap.kt, ap.v};
    std::set<int> seen;
    for (int i = 0; i < 3; ++i) {
      int cast_node = -1;
      const int src = cast_source(operands[i], cast_node);
      if (src < 0 || seen.count(cast_node)) continue;    // one cast feeding two operands stays a kernel of its own
      seen.insert(cast_node);
      *srcs[i] = src;
      interior.push_back(cast_node);
    }
  }
  AttnProblem pr{};
  pr.B = (int)B; pr.H = (int)H; pr.Sq = (int)Sq; pr.Sk = (int)Sk; pr.D = (int)D;
  pr.mode = ap.mode;
  pr.ab_dtype = ap.ab_dtype;
  if (B > 65535 || H > 65535 || Sq > (1 << 24) || Sk > (1 << 24)) return false;
  return attn_tc_supported(pr);
}

void Compiler::plan_attention() {
  attn_plan_.clear();
  attn_absorbed_.clear();
  copy_elided_.clear();
  if (!ctx_->fusion || !ctx_->tensor_cores) return;
  for (int n = 0; n < (int)nodes_.size(); ++n) {
    if (kind_[n] != K_OTHER || nodes_[n].op != BG_OP_MATMUL) continue;
    AttnPlan ap;
    std::vector<int> interior;
    if (!match_attention(n, ap, interior)) continue;
    // result -> PERMUTE (head dim stays last) -> RESHAPE that needs a dense copy, each with one consumer:
    // the kernel stores its rows at the copy's addresses and the copy unit disappears
    const Node& fin = nodes_[n];
    ap.out_stride[0] = fin.shape[1] * fin.shape[2] * fin.shape[3];
    ap.out_stride[1] = fin.shape[2] * fin.shape[3];
    ap.out_stride[2] = fin.shape[3];
    auto only_consumer = [&](int v) {
      std::set<int> c(cons_[v].begin(), cons_[v].end());
      return c.size() == 1 && v != root_ ? *c.begin() : -1;
    };
    const int pm = only_consumer(n);
    const int rs = pm >= 0 && nodes_[pm].op == BG_OP_PERMUTE && kind_[pm] == K_VIEW ? only_consumer(pm) : -1;
    if (rs >= 0 && nodes_[rs].op == BG_OP_RESHAPE && kind_[rs] == K_OTHER && copy_src_.count(rs) && nodes_[pm].iarg[3] == 3 &&
        nodes_[rs].dtype == fin.dtype) {
      int64_t dense[4], run = 1;
      for (int d = 3; d >= 0; --d) { dense[d] = run; run *= nodes_[pm].shape[d]; }
      for (int d = 0; d < 3; ++d) ap.out_stride[nodes_[pm].iarg[d]] = dense[d];
      ap.out_node = rs;
      copy_elided_.insert(rs);
    }
    attn_plan_[n] = ap;
    for (int v : interior) attn_absorbed_.insert(v);
  }
}

void Compiler::emit_attention(int n, int key) {
  const AttnPlan ap = attn_plan_.at(n);
  const Node& fin = nodes_[n];
  AttnProblem tmpl{};
  tmpl.B = (int)fin.shape[0]; tmpl.H = (int)fin.shape[1]; tmpl.Sq = (int)fin.shape[2]; tmpl.D = (int)fin.shape[3];
  const View qv = view_[ap.q], ktv = view_[ap.kt], vv = view_[ap.v];
  tmpl.Sk = (int)ktv.shape[3];
  tmpl.mode = ap.mode;
  tmpl.ab_dtype = ap.ab_dtype;
  tmpl.out_dtype = fin.dtype;
  tmpl.scale = (float)ap.scale_const;
  tmpl.mask_is_bool = ap.mask_is_bool;
  auto operand = [&](const View& v, bool swap_last) {
    AttnOperand o{};
    o.dtype = narrow32_slots_.count(v.slot) ? (int)BG_F32 : v.dtype;   // an fp64 product stored as its fp32 values
    for (int d = 0; d < 4; ++d) o.stride[d] = v.stride[d];
    if (swap_last) std::swap(o.stride[2], o.stride[3]);   // the [B,H,D,Sk] view read as [B,H,Sk,D]
    for (int d = 0; d < 4; ++d)
      if (v.shape[d] == 1) o.stride[d] = 0;
    return o;
  };
  tmpl.q = operand(qv, false);
  tmpl.k = operand(ktv, true);
  tmpl.v = operand(vv, false);
  if (ap.q_src >= 0) tmpl.q.dtype = BG_F32;
  if (ap.kt_src >= 0) tmpl.k.dtype = BG_F32;
  if (ap.v_src >= 0) tmpl.v.dtype = BG_F32;
  int mask_slot = -1;
  int64_t mask_off = 0;
  if (ap.mask >= 0) {
    const View& mv = view_[ap.mask];
    mask_slot = mv.slot;
    mask_off = mv.off * dtype_size(mv.dtype);
    // leading dims align with [B, H] from the right
    const int lead = mv.rank - 2;
    tmpl.mask_sh = lead >= 1 && mv.shape[lead - 1] != 1 ? mv.stride[lead - 1] : 0;
    tmpl.mask_sb = lead >= 2 && mv.shape[lead - 2] != 1 ? mv.stride[lead - 2] : 0;
  }
  int scale_slot = -1;
  int64_t scale_off = 0;
  if (ap.scale_node >= 0) { scale_slot = view_[ap.scale_node].slot; scale_off = view_[ap.scale_node].off * 4; }
  // scratch: Q/K/V^T staging (+ lo parts), tile classes, uniform flag
  AttnProblem sized = tmpl;
  sized.mask = ap.mask >= 0 ? (const void*)1 : nullptr;
  sized.scale_buf = ap.scale_node >= 0 ? (const float*)1 : nullptr;
  int64_t bytes[8];
  attn_scratch_sizes(sized, bytes);
  int scratch_slot[8];
  const int64_t class_bytes = bytes[6];
  PUnit pu;
  for (int i = 0; i < 8; ++i) {
    scratch_slot[i] = bytes[i] > 0 ? new_slot(bytes[i], false, -1) : -1;
    if (scratch_slot[i] >= 0) pu.u.writes.push_back(scratch_slot[i]);
  }
  // an operand whose cast was absorbed is read from the fp32 tensor behind it: same index map, the source's storage
  auto slot_of = [&](const View& v, int src) { return src >= 0 ? view_[src].slot : v.slot; };
  auto off_of = [&](const View& v, int src) {
    if (src < 0 && narrow32_slots_.count(v.slot)) return v.off * (int64_t)4;
    return src >= 0 ? (view_[src].off + v.off) * (int64_t)4 : v.off * (int64_t)dtype_size(v.dtype);
  };
  const int out_node = ap.out_node >= 0 ? ap.out_node : n;
  tmpl.out_sb = ap.out_stride[0]; tmpl.out_sh = ap.out_stride[1]; tmpl.out_ss = ap.out_stride[2];
  const int sq = slot_of(qv, ap.q_src), sk = slot_of(ktv, ap.kt_src), sv = slot_of(vv, ap.v_src), so = view_[out_node].slot;
  const int64_t offq = off_of(qv, ap.q_src), offk = off_of(ktv, ap.kt_src), offv = off_of(vv, ap.v_src);
  pu.order_key = key;
  pu.dep_nodes = {ap.q_src >= 0 ? ap.q_src : ap.q, ap.kt_src >= 0 ? ap.kt_src : ap.kt, ap.v_src >= 0 ? ap.v_src : ap.v};
  if (ap.mask >= 0) pu.dep_nodes.push_back(ap.mask);
  if (ap.scale_node >= 0) pu.dep_nodes.push_back(ap.scale_node);
  pu.out_nodes = {out_node};
  pu.u.name = std::string(ap.mode == 1 ? "attention_tc_3xtf32" : "attention_tc") + (ap.mask >= 0 ? (ap.mask_is_bool ? "+boolmask" : "+mask") : "") +
              (ap.out_node >= 0 ? "+merge" : "") + "[" + dtype_name(fin.dtype) + "]";
  pu.u.launches = 4 + (ap.mask >= 0) + (ap.scale_node >= 0);
  // a 3xTF32 result that only feeds split products (the output projection) leaves the kernel as their operand planes
  int planes_hi = -1, planes_lo = -1;
  if (ap.mode == 1 && feeds_only_split_gemms(out_node)) {
    const int64_t n_out = nodes_[out_node].numel();
    planes_hi = new_slot(n_out * 4, false, -1); planes_lo = new_slot(n_out * 4, false, -1);
    pu.u.writes.push_back(planes_hi); pu.u.writes.push_back(planes_lo);
    publish_planes(out_node, planes_hi, planes_lo, (int)punits_.size());
    pu.u.name += "+split";
  }
  cp_->uses_wait_status = true;
  pu.u.fn = [=](Run& r) {
    AttnProblem a = tmpl;
    if (planes_hi >= 0) { a.planes_hi = r.ptr[planes_hi]; a.planes_lo = r.ptr[planes_lo]; }
    a.q.ptr = reinterpret_cast<char*>(r.ptr[sq]) + offq;
    a.k.ptr = reinterpret_cast<char*>(r.ptr[sk]) + offk;
    a.v.ptr = reinterpret_cast<char*>(r.ptr[sv]) + offv;
    a.mask = mask_slot >= 0 ? reinterpret_cast<char*>(r.ptr[mask_slot]) + mask_off : nullptr;
    a.scale_buf = scale_slot >= 0 ? reinterpret_cast<const float*>(reinterpret_cast<char*>(r.ptr[scale_slot]) + scale_off) : nullptr;
    a.out = r.ptr[so];
    void* scratch[8];
    for (int i = 0; i < 8; ++i) scratch[i] = scratch_slot[i] >= 0 ? r.ptr[scratch_slot[i]] : nullptr;
    // a multiplier bound by handle is examined once; its "one repeated value" flag is kept with the handle
    bool check_uniform = a.scale_buf != nullptr;
    if (a.scale_buf && scale_slot >= 0 && r.from_handle[scale_slot]) {
      bool fresh = false;
      int* flag = uniform_flag_for(r.ctx, a.scale_buf, &fresh);
      if (flag) { scratch[7] = flag; check_uniform = fresh; }
    }
    // likewise the tile classes of a mask bound by handle are computed once and kept with the handle
    bool classify_mask = a.mask != nullptr;
    if (a.mask && mask_slot >= 0 && r.from_handle[mask_slot] && a.mask_sb == 0 && a.mask_sh == 0 && class_bytes > 0) {
      bool fresh = false;
      void* kept = mask_classes_for(r.ctx, a.mask, class_bytes, a.Sq, a.Sk, a.mode == 1 ? 64 : 128, a.mask_is_bool, &fresh);
      if (kept) { scratch[6] = kept; classify_mask = fresh; }
    }
    cudaError_t e = launch_attention_tc(a, scratch, check_uniform, classify_mask, r.ctx->d_status, r.ctx->stream);
    return e == cudaSuccess ? (int)BG_OK : cuda_fail(r.ctx, e, "attention launch");
  };
  add_unit(std::move(pu));
}

void Compiler::emit_matmul(int n, int key) {
  const Node& t = nodes_[n];
  if (t.in.size() != 2) err(BG_ERR_INVALID, "MATMUL: two inputs required");
  const int a = resolve(t.in[0]), b = resolve(t.in[1]);
  View av = view_[a], bv = view_[b];
  if (av.is_const || bv.is_const) err(BG_ERR_UNSUPPORTED, "MATMUL with a scalar constant operand");
  if (av.rank == 0 || bv.rank == 0) err(BG_ERR_INVALID, "MATMUL: 0-d operands");
  // promote 1-D operands to matrices
  bool a_vec = av.rank == 1, b_vec = bv.rank == 1;
  if (a_vec) { av.rank = 2; av.shape[1] = av.shape[0]; av.stride[1] = av.stride[0]; av.shape[0] = 1; av.stride[0] = 0; }
  if (b_vec) { bv.rank = 2; bv.shape[1] = 1; bv.stride[1] = 0; }
  GemmProblem gp{};
  gp.m = av.shape[av.rank - 2];
  gp.k = av.shape[av.rank - 1];
  gp.n = bv.shape[bv.rank - 1];
  if (bv.shape[bv.rank - 2] != gp.k) err(BG_ERR_INVALID, "MATMUL: inner dimensions do not match");
  gp.a.dtype = av.dtype;
  gp.b.dtype = bv.dtype;
  gp.a.row_stride = av.stride[av.rank - 2];
  gp.a.col_stride = av.stride[av.rank - 1];
  gp.b.row_stride = bv.stride[bv.rank - 2];
  gp.b.col_stride = bv.stride[bv.rank - 1];
  // batch dims: broadcast the leading dims, then collapse neighbours both operands walk densely
  const int ba = av.rank - 2, bb = bv.rank - 2, nb = std::max(ba, bb);
  std::vector<int64_t> bs, as, bsb;
  for (int d = 0; d < nb; ++d) {
    int ia = d - (nb - ba), ib = d - (nb - bb);
    int64_t ea = ia >= 0 ? av.shape[ia] : 1, eb = ib >= 0 ? bv.shape[ib] : 1;
    if (ea != eb && ea != 1 && eb != 1) err(BG_ERR_INVALID, "MATMUL: batch dimensions are not broadcastable");
    int64_t e = std::max(ea, eb);
    if (ea == 0 || eb == 0) e = 0;
    int64_t sa = (ia >= 0 && ea != 1) ? av.stride[ia] : 0, sb = (ib >= 0 && eb != 1) ? bv.stride[ib] : 0;
    if (e == 1) continue;
    if (!bs.empty() && as.back() == sa * e && bsb.back() == sb * e) { bs.back() *= e; as.back() = sa; bsb.back() = sb; }
    else { bs.push_back(e); as.push_back(sa); bsb.push_back(sb); }
  }
  if (bs.size() > 4) err(BG_ERR_UNSUPPORTED, "MATMUL: more than four non-collapsible batch dimensions");
  gp.n_batch_dims = (int)bs.size();
  int64_t nbatch = 1;
  for (size_t d = 0; d < bs.size(); ++d) { gp.batch_shape[d] = bs[d]; gp.a.batch_stride[d] = as[d]; gp.b.batch_stride[d] = bsb[d]; nbatch *= bs[d]; }
  if (t.numel() != nbatch * (a_vec ? 1 : gp.m) * (b_vec ? 1 : gp.n)) err(BG_ERR_INVALID, "MATMUL: declared shape does not match the operands");
  gp.c_dtype = t.dtype;
  own_slot(n);
  const int sa = av.slot, sb = bv.slot, sc = view_[n].slot;
  const int64_t offa = av.off * dtype_size(av.dtype), offb = bv.off * dtype_size(bv.dtype);
  // ---- tensor-core path -------------------------------------------------------------
  // 2-D problems whose operands are (or can be copied into) dense K-major matrices:
  //   f16 x f16 / bf16 x bf16 -> tcgen05 kind::f16;   f32 x f32 -> 3xTF32;
  //   fp64 results whose values all derive from fp32 data -> 3xTF32 with an fp64 store.
  {
    const int mode = tc_mode(n);   // 0: 16-bit operands, 1: 3xTF32
    const int ab = mode == 0 ? av.dtype : BG_F32;
    if (mode >= 0) {
      const int64_t M = gp.m, N = gp.n, K = gp.k;
      // operand layouts: A wants [M,K] dense, B wants [N,K] dense (i.e. the [K,N] view with unit stride along K)
      const bool a_dense = gp.a.col_stride == 1 && gp.a.row_stride == K;
      const bool b_kmajor = gp.b.row_stride == 1 && gp.b.col_stride == K;
      const int esa = dtype_size(av.dtype), esb = dtype_size(bv.dtype);
      int a_src = av.slot, b_src = bv.slot;
      int64_t a_off = offa, b_off = offb;
      PUnit pu;
      pu.order_key = key;
      pu.dep_nodes = {a, b};
      pu.out_nodes = {n};
      // operands whose fp32 -> 16-bit cast was absorbed (plan_gemm_casts): read the fp32 tensor, convert here
      int a_f32 = -1, b_f32 = -1;
      {
        auto it = gemm_cast_src_.find(n);
        if (it != gemm_cast_src_.end()) { a_f32 = it->second.first; b_f32 = it->second.second; }
      }
      int a_conv = -1, b_conv = -1;
      bool b_f32_leaf = false;
      if (a_f32 >= 0) {
        // the activation is converted by a unit of its own (its time shows up beside the GEMM's, not inside it)
        const View& sv = view_[a_f32];
        const int f32_slot = sv.slot;
        const int src_dt = sv.dtype;                         // fp32, or float64
        const int64_t f32_off = (sv.off + av.off) * dtype_size(src_dt);
        const auto ckey = std::make_tuple(f32_slot, f32_off, M * K, ab);
        auto chit = conv_memo_.find(ckey);
        if (chit != conv_memo_.end()) {
          // another GEMM of this plan already converts the same activation
          a_conv = chit->second.first;
          pu.dep_punits.push_back(chit->second.second);
          pu.u.reads.push_back(a_conv);
          a_src = a_conv; a_off = 0;
          pu.dep_nodes.erase(pu.dep_nodes.begin());
        } else {
        a_conv = new_slot(M * K * 2, false, -1);
        conv_memo_[ckey] = {a_conv, (int)punits_.size()};
        PUnit cu;
        cu.order_key = key;
        cu.dep_nodes = {a_f32};
        cu.u.writes.push_back(a_conv);
        cu.u.name = std::string("convert16[") + dtype_name(ab) + "]";
        const int conv_slot = a_conv;
        cu.u.fn = [=](Run& r) {
          cudaError_t e = launch_convert16(reinterpret_cast<char*>(r.ptr[f32_slot]) + f32_off, src_dt, r.ptr[conv_slot], M * K, ab,
                                           r.ctx->stream);
          return e == cudaSuccess ? (int)BG_OK : cuda_fail(r.ctx, e, "operand conversion launch");
        };
        pu.dep_punits.push_back((int)punits_.size());
        add_unit(std::move(cu));
        pu.u.reads.push_back(a_conv);
        a_src = a_conv; a_off = 0;
        pu.dep_nodes.erase(pu.dep_nodes.begin());      // A now comes from the conversion unit
        }
      }
      if (b_f32 >= 0) {
        const View& sv = view_[b_f32];
        b_src = sv.slot; b_off = (sv.off + bv.off) * 4;
        b_f32_leaf = cp_->slots[b_src].external;
        if (!b_f32_leaf) { b_conv = new_slot(N * K * 2, false, -1); pu.u.writes.push_back(b_conv); }
        for (int& dn : pu.dep_nodes) if (dn == b) dn = b_f32;
      }
      int a_copy = -1, b_copy = -1;
      StridedView ta{}, tb{};
      if (!a_dense) {
        a_copy = new_slot(M * K * esa, false, -1);
        pu.u.writes.push_back(a_copy);
        ta.dtype = av.dtype; ta.rank = 2; ta.shape[0] = M; ta.shape[1] = K; ta.stride[0] = gp.a.row_stride; ta.stride[1] = gp.a.col_stride;
      }
      if (!b_kmajor) {
        b_copy = new_slot(N * K * esb, false, -1);
        pu.u.writes.push_back(b_copy);
        tb.dtype = bv.dtype; tb.rank = 2; tb.shape[0] = N; tb.shape[1] = K; tb.stride[0] = gp.b.col_stride; tb.stride[1] = gp.b.row_stride;
      }
      int a_hi = -1, a_lo = -1, b_hi = -1, b_lo = -1;
      bool a_shared = false;
      // a weight matrix bound by handle keeps its hi / lo planes with the handle (see split_planes_for)
      const bool b_leaf = mode == 1 && b_copy < 0 && cp_->slots[b_src].external;
      if (mode == 1) {
        const auto a_key = std::make_tuple(a_src, a_off, M * K);
        auto hit = a_copy < 0 ? split_memo_.find(a_key) : split_memo_.end();
        if (hit != split_memo_.end()) {
          // another GEMM of this plan already splits the same operand (q / k / v projections of one LayerNorm output)
          a_hi = hit->second.hi; a_lo = hit->second.lo;
          a_shared = true;
          pu.dep_punits.push_back(hit->second.punit);
          pu.u.reads.push_back(a_hi); pu.u.reads.push_back(a_lo);
        } else {
          a_hi = new_slot(M * K * 4, false, -1); a_lo = new_slot(M * K * 4, false, -1);
          pu.u.writes.push_back(a_hi); pu.u.writes.push_back(a_lo);
          if (a_copy < 0) split_memo_[a_key] = {a_hi, a_lo, (int)punits_.size()};
        }
        if (!b_leaf) {
          b_hi = new_slot(N * K * 4, false, -1); b_lo = new_slot(N * K * 4, false, -1);
          pu.u.writes.push_back(b_hi); pu.u.writes.push_back(b_lo);
        }
      }
      const bool narrow = mode == 1 && narrow_store(n);
      const int a_dt = av.dtype, b_dt = bv.dtype, c_dt = narrow ? BG_F32 : t.dtype;
      auto epi = std::make_shared<TcEpilogue>();
      tc_epilogues_[n] = epi;
      std::string epi_name;
      auto ep_it = epi_plan_.find(n);
      if (ep_it != epi_plan_.end()) {
        const EpiPlan& ep = ep_it->second;
        epi->out_slot = view_[ep.final_node].slot;
        epi->out_dtype = nodes_[ep.final_node].dtype;
        epi->act = ep.act;
        epi->round_acc = ep.round_acc;
        epi->wide = ep.wide;
        if (ep.bias_node >= 0) {
          const View& bvw = view_[ep.bias_node];
          epi->bias_slot = bvw.slot;
          epi->bias_off = bvw.off * dtype_size(bvw.dtype);
          epi->bias_dtype = bvw.dtype;
          pu.dep_nodes.push_back(ep.bias_node);
          epi_name += "+bias";
        }
        if (ep.act == TC_ACT_RELU) epi_name += "+relu";
        if (ep.act == TC_ACT_GELU) epi_name += "+gelu";
        pu.out_nodes = {ep.final_node};
      }
      if (narrow) {
        if (epi->out_slot >= 0) epi->out_dtype = BG_F32;
        narrow32_slots_.insert(view_[pu.out_nodes[0]].slot);
        epi_name += "+f32store";
      }
      // a result that only feeds split products leaves this unit as their operand planes
      int out_hi = -1, out_lo = -1;
      if (mode == 1 && N % 8 == 0 && !gemm_group_of_.count(n) && feeds_only_split_gemms(pu.out_nodes[0])) {   // rows of N: whole 32-byte stores
        out_hi = new_slot(M * N * 4, false, -1); out_lo = new_slot(M * N * 4, false, -1);
        pu.u.writes.push_back(out_hi); pu.u.writes.push_back(out_lo);
        publish_planes(pu.out_nodes[0], out_hi, out_lo, (int)punits_.size());
        epi_name += "+split";
      }
      pu.u.launches = 1 + (a_copy >= 0) + (b_copy >= 0) + (mode == 1 ? (a_shared ? 0 : 1) + 1 : 0) + (b_f32 >= 0);
      pu.u.name = std::string(mode == 0 ? "gemm_tc" : "gemm_tc_3xtf32") + epi_name + "[" + dtype_name(t.dtype) + "]";
      // member of a joint launch: every member but the last only prepares; the last one launches and produces all results
      std::shared_ptr<GroupRun> grun;
      int gidx = 0, gcount = 1;
      {
        auto gi = gemm_group_of_.find(n);
        if (gi != gemm_group_of_.end() && a_copy < 0) {
          GemmGroup& G = gemm_groups_[gi->second];
          grun = G.run;
          gcount = (int)G.members.size();
          gidx = (int)(std::find(G.members.begin(), G.members.end(), n) - G.members.begin());
          const int my_final = pu.out_nodes[0];
          grun->epi[gidx] = epi;
          grun->sc_slot[gidx] = sc;
          grun->c_dt[gidx] = c_dt;
          for (int w : pu.u.writes) G.keep_slots.push_back(w);
          if (gidx + 1 < gcount) {
            G.finals.push_back(my_final);
            G.punits.push_back((int)punits_.size());
            pu.out_nodes.clear();
            pu.u.launches -= 1;
            pu.u.name = std::string("gemm_operands[") + dtype_name(t.dtype) + "]";
          } else {
            for (int f : G.finals) pu.out_nodes.push_back(f);
            for (int u : G.punits) pu.dep_punits.push_back(u);
            for (int w : G.keep_slots) pu.u.reads.push_back(w);
            pu.u.name += " x" + std::to_string(gcount);
          }
        }
      }
      cp_->uses_wait_status = true;
      const int sc_slot = sc;
      pu.u.fn = [=](Run& r) {
        cudaStream_t st = r.ctx->stream;
        const void* pa = reinterpret_cast<char*>(r.ptr[a_src]) + a_off;
        const void* pb = reinterpret_cast<char*>(r.ptr[b_src]) + b_off;
        cudaError_t e = cudaSuccess;
        if (a_copy >= 0) {
          StridedView v = ta; v.ptr = pa;
          e = launch_strided_copy(v, r.ptr[a_copy], M * K, st);
          if (e != cudaSuccess) return cuda_fail(r.ctx, e, "gemm operand copy");
          pa = r.ptr[a_copy];
        }
        if (b_copy >= 0) {
          StridedView v = tb; v.ptr = pb;
          e = launch_strided_copy(v, r.ptr[b_copy], N * K, st);
          if (e != cudaSuccess) return cuda_fail(r.ctx, e, "gemm operand copy");
          pb = r.ptr[b_copy];
        }
        TcGemm g{};
        g.M = M; g.N = N; g.K = K;
        g.ab_dtype = ab;
        void* tmp_planes = nullptr;     // hi / lo planes of a B operand that is neither a slot nor kept with a handle
        if (mode == 1) {
          if (!a_shared) e = launch_tf32_split(pa, a_dt, (float*)r.ptr[a_hi], (float*)r.ptr[a_lo], M * K, K, st);
          float* bh = b_leaf ? nullptr : (float*)r.ptr[b_hi];
          float* bl = b_leaf ? nullptr : (float*)r.ptr[b_lo];
          bool split_b = true;
          if (b_leaf) {
            bool fresh = false;
            float* kept = r.from_handle[b_src] ? split_planes_for(r.ctx, pb, N * K, b_dt, &fresh) : nullptr;
            if (kept) { bh = kept; bl = kept + N * K; split_b = fresh; }
            else {
              if (int rc = dev_alloc(r.ctx, 2 * N * K * 4, &tmp_planes)) return rc;
              bh = reinterpret_cast<float*>(tmp_planes); bl = bh + N * K;
            }
          }
          if (e == cudaSuccess && split_b) e = launch_tf32_split(pb, b_dt, bh, bl, N * K, K, st);
          if (e != cudaSuccess) { if (tmp_planes) dev_free(r.ctx, tmp_planes, 2 * N * K * 4); return cuda_fail(r.ctx, e, "tf32 split launch"); }
          g.A = r.ptr[a_hi]; g.A_lo = r.ptr[a_lo]; g.B = bh; g.B_lo = bl;
        } else {
          if (e == cudaSuccess && b_f32 >= 0) {
            void* dst = nullptr;
            bool convert = true;
            if (b_f32_leaf) {
              // a weight bound by handle keeps its 16-bit copy with the handle
              bool fresh = false;
              dst = r.from_handle[b_src] ? cast_copy_for(r.ctx, pb, N * K * 2, ab, &fresh) : nullptr;
              if (dst) convert = fresh;
              else {
                if (int rc = dev_alloc(r.ctx, N * K * 2, &tmp_planes)) return rc;
                dst = tmp_planes;
              }
            } else {
              dst = r.ptr[b_conv];
            }
            if (convert) e = launch_convert16(pb, BG_F32, dst, N * K, ab, st);
            pb = dst;
          }
          if (e != cudaSuccess) { if (tmp_planes) dev_free(r.ctx, tmp_planes, N * K * 2); return cuda_fail(r.ctx, e, "operand conversion launch"); }
          g.A = pa; g.B = pb;
        }
        g.C = r.ptr[epi->out_slot >= 0 ? epi->out_slot : sc_slot];
        g.c_dtype = epi->out_slot >= 0 ? epi->out_dtype : c_dt;
        if (epi->bias_slot >= 0) {
          g.bias = reinterpret_cast<char*>(r.ptr[epi->bias_slot]) + epi->bias_off;
          g.bias_dtype = epi->bias_dtype;
        }
        g.act = epi->act;
        g.round_acc = epi->round_acc;
        g.wide = epi->wide;
        if (out_hi >= 0) { g.planes_hi = r.ptr[out_hi]; g.planes_lo = r.ptr[out_lo]; }
        const size_t tmp_bytes = mode == 1 ? 2 * N * K * 4 : N * K * 2;
        if (grun) {
          // a run that stopped between the members leaves their temporary planes behind: the next run's
          // first member releases them
          if (gidx == 0)
            for (int i = 0; i < gcount; ++i)
              if (grun->tmp[i]) { dev_free(r.ctx, grun->tmp[i], grun->tmp_bytes[i]); grun->tmp[i] = nullptr; }
          grun->g[gidx] = g;
          grun->tmp[gidx] = tmp_planes;
          grun->tmp_bytes[gidx] = tmp_bytes;
          if (gidx + 1 < gcount) return (int)BG_OK;
          for (int i = 0; i < gcount; ++i) {
            const TcEpilogue& ei = *grun->epi[i];
            grun->g[i].C = r.ptr[ei.out_slot >= 0 ? ei.out_slot : grun->sc_slot[i]];
            grun->g[i].c_dtype = ei.out_slot >= 0 ? ei.out_dtype : grun->c_dt[i];
            grun->g[i].bias = ei.bias_slot >= 0 ? reinterpret_cast<char*>(r.ptr[ei.bias_slot]) + ei.bias_off : nullptr;
          }
          e = launch_gemm_tc_group(grun->g, gcount, r.ctx->d_status, st);
          for (int i = 0; i < gcount; ++i)
            if (grun->tmp[i]) { dev_free(r.ctx, grun->tmp[i], grun->tmp_bytes[i]); grun->tmp[i] = nullptr; }
          return e == cudaSuccess ? (int)BG_OK : cuda_fail(r.ctx, e, "tensor-core gemm launch");
        }
        e = launch_gemm_tc(g, r.ctx->d_status, st);
        if (tmp_planes) dev_free(r.ctx, tmp_planes, tmp_bytes);    // stream-ordered: released after the GEMM has run
        return e == cudaSuccess ? (int)BG_OK : cuda_fail(r.ctx, e, "tensor-core gemm launch");
      };
      tc_unit_of_[n] = (int)punits_.size();
      add_unit(std::move(pu));
      return;
    }
  }
  {
    int splits = 0;
    int64_t partial_bytes = 0;
    if (!a_vec && !b_vec && small_gemm(n, &splits, &partial_bytes) && gemm_small_plan(gp, ctx_->sm_count, &splits, &partial_bytes)) {
      PUnit pu;
      pu.order_key = key;
      pu.dep_nodes = {a, b};
      pu.out_nodes = {n};
      int out_slot = sc, bias_slot = -1, act = TC_ACT_NONE;
      int64_t bias_off = 0;
      std::string epi_name;
      auto ep_it = epi_plan_.find(n);
      if (ep_it != epi_plan_.end()) {
        const EpiPlan& ep = ep_it->second;
        out_slot = view_[ep.final_node].slot;
        act = ep.act;
        if (ep.bias_node >= 0) {
          const View& bvw = view_[ep.bias_node];
          bias_slot = bvw.slot;
          bias_off = bvw.off * 4;
          pu.dep_nodes.push_back(ep.bias_node);
          epi_name += "+bias";
        }
        if (act == TC_ACT_RELU) epi_name += "+relu";
        pu.out_nodes = {ep.final_node};
      }
      const int part_slot = partial_bytes > 0 ? new_slot(partial_bytes, false, -1) : -1;
      if (part_slot >= 0) pu.u.writes.push_back(part_slot);
      pu.u.name = std::string("gemm_small") + epi_name + "[float32]";
      pu.u.fn = [=](Run& r) {
        GemmProblem p = gp;
        p.a.ptr = reinterpret_cast<char*>(r.ptr[sa]) + offa;
        p.b.ptr = reinterpret_cast<char*>(r.ptr[sb]) + offb;
        p.c = r.ptr[out_slot];
        const void* bias = bias_slot >= 0 ? reinterpret_cast<char*>(r.ptr[bias_slot]) + bias_off : nullptr;
        cudaError_t e = launch_gemm_small(p, bias, act, part_slot >= 0 ? r.ptr[part_slot] : nullptr, r.ctx->gemm_counters, splits,
                                          r.ctx->stream);
        return e == cudaSuccess ? (int)BG_OK : cuda_fail(r.ctx, e, "small gemm launch");
      };
      add_unit(std::move(pu));
      return;
    }
  }
  PUnit pu;
  pu.order_key = key;
  pu.dep_nodes = {a, b};
  pu.out_nodes = {n};
  pu.u.name = std::string("gemm_simt[") + dtype_name(t.dtype) + "]";
  pu.u.fn = [=](Run& r) {
    GemmProblem p = gp;
    p.a.ptr = reinterpret_cast<char*>(r.ptr[sa]) + offa;
    p.b.ptr = reinterpret_cast<char*>(r.ptr[sb]) + offb;
    p.c = r.ptr[sc];
    cudaError_t e = launch_gemm_simt(p, r.ctx->stream);
    return e == cudaSuccess ? (int)BG_OK : cuda_fail(r.ctx, e, "gemm launch");
  };
  add_unit(std::move(pu));
}

void Compiler::emit_index(int n, int key) {
  const Node& t = nodes_[n];
  if (t.in.size() != 2) err(BG_ERR_INVALID, "INDEX: two inputs required");
  const int x = resolve(t.in[0]), ix = resolve(t.in[1]);
  const View xv = view_[x], iv = view_[ix];
  if (iv.dtype != BG_I64) err(BG_ERR_INVALID, "INDEX: index dtype must be int64");
  if (xv.rank != iv.rank || xv.rank == 0) err(BG_ERR_INVALID, "INDEX: source and index must have the same nonzero rank");
  const int dim = (int)t.iarg[0];
  if (dim < 0 || dim >= xv.rank) err(BG_ERR_INVALID, "INDEX: dimension out of range");
  for (int d = 0; d < xv.rank; ++d)
    if (d != dim && iv.shape[d] > xv.shape[d]) err(BG_ERR_INVALID, "INDEX: index extent exceeds source extent");
  if (!xv.contiguous() || !iv.contiguous() || xv.is_const || iv.is_const) err(BG_ERR_UNSUPPORTED, "INDEX: operands must be dense tensors");
  own_slot(n);
  const int sx = xv.slot, si = iv.slot, so = view_[n].slot, es = dtype_size(xv.dtype), rank = xv.rank;
  const int64_t offx = xv.off * es, offi = iv.off * 8;
  std::vector<int64_t> xs(xv.shape, xv.shape + rank), is(iv.shape, iv.shape + rank);
  cp_->uses_status = true;
  PUnit pu;
  pu.order_key = key;
  pu.dep_nodes = {x, ix};
  pu.out_nodes = {n};
  pu.u.name = "gather[INDEX]";
  pu.u.fn = [=](Run& r) {
    cudaError_t e = launch_gather(reinterpret_cast<char*>(r.ptr[sx]) + offx,
                                  reinterpret_cast<const int64_t*>(reinterpret_cast<char*>(r.ptr[si]) + offi), r.ptr[so], es, rank,
                                  xs.data(), is.data(), dim, r.ctx->d_status, r.ctx->stream);
    return e == cudaSuccess ? (int)BG_OK : cuda_fail(r.ctx, e, "gather launch");
  };
  add_unit(std::move(pu));
}

// TRIL / TRIU / FLIP / CUMSUM (one input) and CONCAT (several): strided views in, one dense tensor out.
void Compiler::emit_shape_op(int n, int key) {
  const Node& t = nodes_[n];
  const int n_in = (int)t.in.size();
  if (t.op == BG_OP_CONCAT) { if (n_in < 1) err(BG_ERR_INVALID, "CONCAT: no inputs"); }
  else if (n_in != 1) err(BG_ERR_INVALID, std::string(op_name(t.op)) + ": one input required");
  struct Src { int slot; int64_t off_bytes; StridedView v; bool is_fill; PlaceFill fill; };
  std::vector<Src> srcs;
  std::vector<int> deps;
  for (int k = 0; k < n_in; ++k) {
    const int x = resolve(t.in[k]);
    const View& xv = view_[x];
    if (xv.is_const && t.op != BG_OP_CONCAT) err(BG_ERR_UNSUPPORTED, std::string(op_name(t.op)) + " of a scalar constant");
    Src sc{};
    sc.is_fill = xv.is_const;
    if (xv.is_const) {
      // the constant converted to its own dtype first, as the reference materialises it before concatenating
      sc.fill.is_int = !dtype_is_float(xv.dtype);
      sc.fill.f = xv.dtype == BG_F32 ? (double)(float)xv.cf : xv.cf;
      sc.fill.n = xv.dtype == BG_BOOL ? (xv.ci != 0) : xv.ci;
    }
    sc.slot = xv.slot;
    sc.off_bytes = xv.off * dtype_size(xv.dtype);
    sc.v.dtype = xv.dtype;
    sc.v.rank = xv.rank;
    for (int d = 0; d < xv.rank; ++d) { sc.v.shape[d] = xv.shape[d]; sc.v.stride[d] = xv.shape[d] == 1 ? 0 : xv.stride[d]; }
    srcs.push_back(sc);
    if (!xv.is_const) deps.push_back(x);
  }
  const int rank = t.rank;
  const int64_t a0 = t.iarg[0];
  const View& x0 = view_[resolve(t.in[0])];
  const bool ordering = t.op == BG_OP_SORT_INDICES || t.op == BG_OP_TOPK_INDICES;
  if (t.op != BG_OP_CONCAT) {
    if (x0.rank != rank) err(BG_ERR_INVALID, std::string(op_name(t.op)) + ": result rank differs from the input's");
    for (int d = 0; d < rank; ++d)
      if (x0.shape[d] != t.shape[d] && !(t.op == BG_OP_TOPK_INDICES && d == a0))
        err(BG_ERR_INVALID, std::string(op_name(t.op)) + ": result shape differs from the input's");
  }
  int64_t keep = 0;
  if (ordering) {
    if (rank == 0 || a0 < 0 || a0 >= rank) err(BG_ERR_INVALID, std::string(op_name(t.op)) + ": axis out of range");
    if (t.dtype != BG_I64) err(BG_ERR_INVALID, std::string(op_name(t.op)) + ": positions are int64");
    if (x0.shape[a0] > kSortMaxLine)
      err(BG_ERR_UNSUPPORTED, std::string(op_name(t.op)) + ": lines longer than " + std::to_string(kSortMaxLine) + " elements are not supported");
    keep = t.op == BG_OP_SORT_INDICES ? x0.shape[a0] : t.iarg[1];
    if (t.op == BG_OP_TOPK_INDICES) {
      if (keep < 0 || keep > x0.shape[a0] || t.shape[a0] != keep) err(BG_ERR_INVALID, "TOPK_INDICES: k does not match the shapes");
      if (!t.iarg[3]) err(BG_ERR_UNSUPPORTED, "TOPK_INDICES: sorted=False has no defined order to reproduce");
    }
  }
  if ((t.op == BG_OP_TRIL || t.op == BG_OP_TRIU)) {
    if (rank < 2) err(BG_ERR_INVALID, "TRIL/TRIU: at least two dimensions required");
    if (x0.dtype != t.dtype) err(BG_ERR_INVALID, "TRIL/TRIU: dtype must be preserved");
  }
  if (t.op == BG_OP_FLIP) {
    if (a0 < 0 || a0 >= rank) err(BG_ERR_INVALID, "FLIP: axis out of range");
    if (x0.dtype != t.dtype) err(BG_ERR_INVALID, "FLIP: dtype must be preserved");
  }
  if (t.op == BG_OP_CUMSUM && (a0 < 0 || a0 >= rank)) err(BG_ERR_INVALID, "CUMSUM: axis out of range");
  std::vector<int64_t> axis_off;
  if (t.op == BG_OP_CONCAT) {
    if (a0 < 0 || a0 >= rank) err(BG_ERR_INVALID, "CONCAT: axis out of range");
    int64_t total = 0;
    for (const Src& sc : srcs) {
      if (sc.v.rank != rank) err(BG_ERR_INVALID, "CONCAT: inputs must have the result's rank");
      for (int d = 0; d < rank; ++d)
        if (d != a0 && sc.v.shape[d] != t.shape[d]) err(BG_ERR_INVALID, "CONCAT: input extents off the axis must match the result");
      axis_off.push_back(total);
      total += sc.v.shape[a0];
    }
    if (total != t.shape[a0]) err(BG_ERR_INVALID, "CONCAT: input extents along the axis do not add up to the result's");
  }
  own_slot(n);
  const int so = view_[n].slot, op = t.op, out_dt = t.dtype;
  const int64_t numel = t.numel();
  const int reverse = (int)t.iarg[1];      // CUMSUM: reverse; SORT_INDICES: descending
  const int largest = (int)t.iarg[2];
  std::vector<int64_t> oshape(t.shape, t.shape + rank);
  PUnit pu;
  pu.order_key = key;
  pu.dep_nodes = deps;
  pu.out_nodes = {n};
  pu.u.launches = op == BG_OP_CONCAT ? n_in : 1;
  pu.u.name = op == BG_OP_CONCAT ? "place[CONCAT]" : (op == BG_OP_CUMSUM ? "scan[CUMSUM]"
              : (ordering ? std::string("sort_lines[") + op_name(op) + "]" : std::string("index_map[") + op_name(op) + "]"));
  pu.u.fn = [=](Run& r) {
    cudaError_t e = cudaSuccess;
    for (size_t k = 0; k < srcs.size() && e == cudaSuccess; ++k) {
      StridedView v = srcs[k].v;
      v.ptr = srcs[k].is_fill ? nullptr : reinterpret_cast<char*>(r.ptr[srcs[k].slot]) + srcs[k].off_bytes;
      switch (op) {
        case BG_OP_TRIL: e = launch_tri(v, r.ptr[so], numel, 0, a0, r.ctx->stream); break;
        case BG_OP_TRIU: e = launch_tri(v, r.ptr[so], numel, 1, a0, r.ctx->stream); break;
        case BG_OP_FLIP: e = launch_flip(v, r.ptr[so], numel, (int)a0, r.ctx->stream); break;
        case BG_OP_CUMSUM: e = launch_cumsum(v, r.ptr[so], out_dt, (int)a0, reverse, r.ctx->stream); break;
        case BG_OP_SORT_INDICES:
          e = launch_sort_lines(v, reinterpret_cast<int64_t*>(r.ptr[so]), (int)a0, reverse, keep, r.ctx->stream); break;
        case BG_OP_TOPK_INDICES:
          e = launch_sort_lines(v, reinterpret_cast<int64_t*>(r.ptr[so]), (int)a0, largest, keep, r.ctx->stream); break;
        default: e = launch_place(v, r.ptr[so], out_dt, oshape.data(), (int)a0, axis_off[k], r.ctx->stream, srcs[k].is_fill ? &srcs[k].fill : nullptr); break;
      }
    }
    return e == cudaSuccess ? (int)BG_OK : cuda_fail(r.ctx, e, "data-movement kernel launch");
  };
  add_unit(std::move(pu));
}

// SCATTER: dense copy of the target, then one thread per index entry stores its source value.
void Compiler::emit_scatter(int n, int key) {
  const Node& t = nodes_[n];
  if (t.in.size() != 3) err(BG_ERR_INVALID, "SCATTER: target, index and source inputs required");
  const int tg = resolve(t.in[0]), ix = resolve(t.in[1]), sr = resolve(t.in[2]);
  const View tv = view_[tg], iv = view_[ix], sv = view_[sr];
  const int rank = t.rank, dim = (int)t.iarg[0];
  if (rank == 0 || tv.rank != rank || iv.rank != rank) err(BG_ERR_INVALID, "SCATTER: target and index must have the same nonzero rank");
  if (dim < 0 || dim >= rank) err(BG_ERR_INVALID, "SCATTER: dimension out of range");
  if (iv.dtype != BG_I64) err(BG_ERR_INVALID, "SCATTER: index dtype must be int64");
  if (tv.dtype != t.dtype || sv.dtype != t.dtype) err(BG_ERR_INVALID, "SCATTER: target, source and result share one dtype");
  for (int d = 0; d < rank; ++d) {
    if (tv.shape[d] != t.shape[d]) err(BG_ERR_INVALID, "SCATTER: result shape must equal the target's");
    if (iv.shape[d] > tv.shape[d]) err(BG_ERR_INVALID, "SCATTER: index extent exceeds target extent");
  }
  if (tv.is_const || iv.is_const) err(BG_ERR_UNSUPPORTED, "SCATTER: target and index must be tensors");
  if (!iv.contiguous()) err(BG_ERR_UNSUPPORTED, "SCATTER: index must be a dense tensor");
  const bool src_const = sv.is_const;
  if (!src_const) {
    if (sv.rank != rank || !sv.contiguous()) err(BG_ERR_UNSUPPORTED, "SCATTER: source must be a dense tensor of the index's shape or a scalar");
    for (int d = 0; d < rank; ++d)
      if (sv.shape[d] != iv.shape[d]) err(BG_ERR_INVALID, "SCATTER: source shape must equal the index shape");
  }
  // the scalar source in the result's own representation
  unsigned long long bits = 0;
  if (src_const) {
    switch (t.dtype) {
      case BG_F64: { double v = sv.cf; memcpy(&bits, &v, 8); break; }
      case BG_F32: { float v = (float)sv.cf; memcpy(&bits, &v, 4); break; }
      case BG_F16: case BG_BF16: err(BG_ERR_UNSUPPORTED, "SCATTER: scalar sources of 16-bit tensors are not supported");
      case BG_BOOL: bits = sv.ci != 0; break;
      default: bits = (unsigned long long)sv.ci; break;
    }
  }
  own_slot(n);
  const int es = dtype_size(t.dtype);
  const int64_t numel = t.numel();
  const int claim_slot = new_slot(std::max<int64_t>(numel, 1) * 4, false, -1);
  const int st = tv.slot, si = iv.slot, ss = src_const ? -1 : sv.slot, so = view_[n].slot;
  const int64_t off_t = tv.off * es, off_i = iv.off * 8, off_s = src_const ? 0 : sv.off * es;
  StridedView tmpl{};
  tmpl.dtype = tv.dtype;
  tmpl.rank = rank;
  for (int d = 0; d < rank; ++d) { tmpl.shape[d] = tv.shape[d]; tmpl.stride[d] = tv.shape[d] == 1 ? 0 : tv.stride[d]; }
  std::vector<int64_t> oshape(t.shape, t.shape + rank), ishape(iv.shape, iv.shape + rank);
  cp_->uses_status = true;
  PUnit pu;
  pu.order_key = key;
  pu.dep_nodes = {tg, ix};
  if (!src_const) pu.dep_nodes.push_back(sr);
  pu.out_nodes = {n};
  pu.u.writes.push_back(claim_slot);
  pu.u.launches = 3;
  pu.u.name = "scatter[SCATTER]";
  pu.u.fn = [=](Run& r) {
    StridedView v = tmpl;
    v.ptr = reinterpret_cast<char*>(r.ptr[st]) + off_t;
    cudaError_t e = launch_strided_copy(v, r.ptr[so], numel, r.ctx->stream);
    if (e == cudaSuccess)
      e = launch_scatter(reinterpret_cast<const int64_t*>(reinterpret_cast<char*>(r.ptr[si]) + off_i),
                         ss >= 0 ? reinterpret_cast<char*>(r.ptr[ss]) + off_s : nullptr, r.ptr[so],
                         reinterpret_cast<int*>(r.ptr[claim_slot]), es, rank, oshape.data(), ishape.data(), dim, src_const, bits,
                         r.ctx->d_status, r.ctx->stream);
    return e == cudaSuccess ? (int)BG_OK : cuda_fail(r.ctx, e, "scatter launch");
  };
  add_unit(std::move(pu));
}

void Compiler::emit_ce(int n, int key) {
  // iarg: [0] reduction (0 none, 1 mean, 2 sum), [1] ignore_index, [2] batch_rank, [3] bit 0 probability targets,
  // bit 1 class weights as a third input; farg[0] label smoothing
  const Node& t = nodes_[n];
  const bool prob = (t.iarg[3] & 1) != 0, has_w = (t.iarg[3] & 2) != 0;
  if (t.in.size() != (has_w ? 3u : 2u)) err(BG_ERR_INVALID, "CROSS_ENTROPY: inputs are (logits, targets[, class weights])");
  const int x = resolve(t.in[0]), tg = resolve(t.in[1]), wn = has_w ? resolve(t.in[2]) : -1;
  const View xv = view_[x], tv = view_[tg];
  if (xv.dtype != BG_F32 && xv.dtype != BG_F64) err(BG_ERR_UNSUPPORTED, "CROSS_ENTROPY: float32/float64 logits only");
  if (!prob && tv.dtype != BG_I64) err(BG_ERR_UNSUPPORTED, "CROSS_ENTROPY: class-index targets must be int64");
  if (prob && tv.dtype != xv.dtype) err(BG_ERR_UNSUPPORTED, "CROSS_ENTROPY: probability targets must have the logits' dtype");
  if (t.dtype != xv.dtype) err(BG_ERR_INVALID, "CROSS_ENTROPY: output dtype must equal the logits dtype");
  if (!xv.contiguous() || !tv.contiguous() || xv.is_const || tv.is_const) err(BG_ERR_UNSUPPORTED, "CROSS_ENTROPY: operands must be dense tensors");
  if (t.iarg[2] != 0) err(BG_ERR_UNSUPPORTED, "CROSS_ENTROPY: batch_rank must be 0");
  const int reduction = (int)t.iarg[0];
  const int64_t ignore = t.iarg[1];
  const double smoothing = t.farg[0];
  if (!(smoothing >= 0.0 && smoothing <= 1.0)) err(BG_ERR_INVALID, "CROSS_ENTROPY: label smoothing outside [0, 1]");
  int64_t outer, C, inner = 1;
  if (xv.rank == 1) { outer = 1; C = xv.shape[0]; }
  else { outer = xv.shape[0]; C = xv.shape[1]; for (int d = 2; d < xv.rank; ++d) inner *= xv.shape[d]; }
  if (tv.numel() != (prob ? outer * C * inner : outer * inner)) err(BG_ERR_INVALID, "CROSS_ENTROPY: target shape does not match the logits");
  if (C == 0) err(BG_ERR_INVALID, "CROSS_ENTROPY: empty class axis");
  View wv;
  if (has_w) {
    wv = view_[wn];
    if (wv.dtype != xv.dtype) err(BG_ERR_UNSUPPORTED, "CROSS_ENTROPY: class weights must have the logits' dtype");
    if (wv.numel() != C || !wv.contiguous() || wv.is_const) err(BG_ERR_INVALID, "CROSS_ENTROPY: class weights must be a dense [C] tensor");
  }
  own_slot(n);
  const int es = dtype_size(xv.dtype);
  const int64_t npos = outer * inner;
  const int npos_slot = reduction == 0 ? view_[n].slot : new_slot(npos * es, false, -1);
  // the weighted mean divides by the summed weights of the valid targets: one more value per position
  const int selw_slot = (has_w && !prob && reduction == 1) ? new_slot(npos * es, false, -1) : -1;
  const int sx = xv.slot, st = tv.slot, sw = has_w ? wv.slot : -1, so = view_[n].slot, dt = xv.dtype;
  const int64_t offx = xv.off * es, offt = tv.off * dtype_size(tv.dtype), offw = has_w ? wv.off * es : 0;
  cp_->uses_status = true;
  PUnit pu;
  pu.order_key = key;
  pu.dep_nodes = {x, tg};
  if (has_w) pu.dep_nodes.push_back(wn);
  pu.out_nodes = {n};
  pu.u.name = std::string("cross_entropy") + (prob ? "+prob" : "") + (has_w ? "+weight" : "") + (smoothing != 0.0 ? "+smooth" : "");
  pu.u.launches = reduction == 0 ? 1 : 2;
  if (npos_slot != so) pu.u.writes.push_back(npos_slot);
  if (selw_slot >= 0) pu.u.writes.push_back(selw_slot);
  pu.u.fn = [=](Run& r) {
    CeProblem c{};
    c.logits = reinterpret_cast<char*>(r.ptr[sx]) + offx;
    c.targets = reinterpret_cast<char*>(r.ptr[st]) + offt;
    c.weight = sw >= 0 ? reinterpret_cast<char*>(r.ptr[sw]) + offw : nullptr;
    c.per_pos = r.ptr[npos_slot];
    c.sel_w = selw_slot >= 0 ? r.ptr[selw_slot] : nullptr;
    c.dtype = dt;
    c.prob_targets = prob ? 1 : 0;
    c.outer = outer; c.C = C; c.inner = inner; c.ignore_index = ignore;
    c.label_smoothing = smoothing;
    c.status = r.ctx->d_status;
    if (reduction != 0 && ce_small_usable(c)) {
      cudaError_t e1 = launch_ce_small(c, r.ptr[so], reduction, (double)npos, r.ctx->stream);
      return e1 == cudaSuccess ? (int)BG_OK : cuda_fail(r.ctx, e1, "cross entropy launch");
    }
    cudaError_t e = launch_ce_rows(c, r.ctx->stream);
    if (e == cudaSuccess && reduction != 0)
      e = launch_ce_reduce(c.per_pos, prob ? nullptr : reinterpret_cast<const int64_t*>(c.targets), c.sel_w, r.ptr[so], dt, npos, reduction,
                           ignore, (double)npos, r.ctx->stream);
    return e == cudaSuccess ? (int)BG_OK : cuda_fail(r.ctx, e, "cross entropy launch");
  };
  add_unit(std::move(pu));
}

bool Compiler::try_lower() {
  cp_ = std::make_shared<CompiledPlan>();
  punits_.clear();
  nodes_.clear();
  copy_src_.clear();
  tc_epilogues_.clear();
  split_memo_.clear();
  narrow32_slots_.clear();
  conv_memo_.clear();
  tc_unit_of_.clear();
  attn_plan_.clear();
  attn_absorbed_.clear();
  has_f64_leaf_ = false;
  expand();
  simplify();
  build_views();
  if (force_break_.size() != nodes_.size()) force_break_.assign(nodes_.size(), 0);
  analyse();
  const int nn = (int)nodes_.size();
  // group membership lists in node order
  std::map<int, std::vector<int>> groups;
  for (int i = 0; i < nn; ++i)
    if (kind_[i] == K_EW) groups[find(i)].push_back(i);
  plan_attention();
  plan_gemm_casts();
  plan_tc_epilogues(groups);
  plan_gemm_groups();
  // only groups with a materialised member or a tail do any work
  for (auto& kv : groups) {
    const std::vector<int>& mem = kv.second;
    if (absorbed_groups_.count(kv.first)) continue;   // runs as the epilogue of a tensor-core GEMM
    {
      bool in_attention = false;
      for (int m : mem) in_attention |= attn_absorbed_.count(m) != 0;
      if (in_attention) continue;                       // interior of a fused attention
    }
    bool live = tail_of_group_[kv.first] >= 0;
    for (int m : mem) live |= need_mat_[m] != 0;
    if (!live) continue;
    try {
      emit_group(mem, tail_of_group_[kv.first], mem.back());
    } catch (CompileError& ce) {
      if (ce.code != -1) throw;
      // split: stop fusing through the middle member (or drop the tail) and recompile
      if (tail_of_group_[kv.first] >= 0 && mem.size() <= 1) force_break_[mem[0]] = 1;
      else if (tail_of_group_[kv.first] >= 0 && ce.msg.find("row does not fit") != std::string::npos) force_break_[resolve(nodes_[tail_of_group_[kv.first]].in[0])] = 1;
      else if (mem.size() >= 2) force_break_[mem[mem.size() / 2 - 1]] = 1;
      else err(BG_ERR_UNSUPPORTED, "elementwise group cannot be lowered: " + ce.msg);
      return false;
    }
  }
  for (int i = 0; i < nn; ++i) {
    const Node& n = nodes_[i];
    if (attn_absorbed_.count(i)) continue;
    if (kind_[i] == K_OTHER && n.op == BG_OP_MATMUL && attn_plan_.count(i)) { emit_attention(i, i); continue; }
    if (kind_[i] == K_ROW && attached_[i] < 0) {
      int64_t rows, cols;
      View xin;
      bool trailing;
      row_geometry(i, rows, cols, xin, trailing);
      const int x = resolve(n.in[0]);
      if (view_[x].is_const) err(BG_ERR_UNSUPPORTED, std::string(op_name(n.op)) + " of a scalar constant");
      if (trailing) {
        try {
          emit_row_standalone(i, i);
        } catch (CompileError& ce) {
          if (ce.code != -1) throw;
          if (n.op == BG_OP_FUSED_SOFTMAX && view_[x].contiguous()) emit_generic_softmax(i, i);
          else err(BG_ERR_UNSUPPORTED, std::string(op_name(n.op)) + ": " + ce.msg);
        }
      } else if (n.op == BG_OP_FUSED_SOFTMAX) {
        if (!view_[x].contiguous()) err(BG_ERR_UNSUPPORTED, "FUSED_SOFTMAX over a non-trailing axis of a strided view");
        emit_generic_softmax(i, i);
      } else {
        const uint64_t mask = (uint64_t)n.iarg[1];
        bool block = true;
        int lo = -1, hi = -1;
        for (int d = 0; d < nodes_[x].rank; ++d)
          if ((mask >> d) & 1) { if (lo < 0) lo = d; hi = d; }
        for (int d = lo; d <= hi && lo >= 0; ++d)
          if (!((mask >> d) & 1)) block = false;
        if (block && view_[x].contiguous()) emit_generic_reduce(i, i);
        else {
          // permute the view so that the reduced axes trail, then run the row kernel on it
          View pv = view_[x];
          View nv = pv;
          int k = 0;
          for (int d = 0; d < pv.rank; ++d)
            if (!((mask >> d) & 1)) { nv.shape[k] = pv.shape[d]; nv.stride[k] = pv.stride[d]; ++k; }
          for (int d = 0; d < pv.rank; ++d)
            if ((mask >> d) & 1) { nv.shape[k] = pv.shape[d]; nv.stride[k] = pv.stride[d]; ++k; }
          // temporarily present the permuted view as the input's view
          const View saved = view_[x];
          const Node saved_node = nodes_[x];
          view_[x] = nv;
          for (int d = 0; d < nv.rank; ++d) nodes_[x].shape[d] = nv.shape[d];
          Node saved_r = nodes_[i];
          uint64_t m2 = 0;
          int kept = 0;
          for (int d = 0; d < pv.rank; ++d) kept += !((mask >> d) & 1);
          for (int d = kept; d < pv.rank; ++d) m2 |= 1ull << d;
          nodes_[i].iarg[1] = (int64_t)m2;
          try {
            emit_row_standalone(i, i);
          } catch (CompileError& ce) {
            view_[x] = saved; nodes_[x] = saved_node; nodes_[i] = saved_r;
            if (ce.code != -1) throw;
            err(BG_ERR_UNSUPPORTED, "REDUCE: " + ce.msg);
          }
          view_[x] = saved;
          nodes_[x] = saved_node;
          nodes_[i] = saved_r;
        }
      }
    } else if (kind_[i] == K_OTHER) {
      switch (n.op) {
        case BG_OP_MATMUL: emit_matmul(i, i); break;
        case BG_OP_INDEX: emit_index(i, i); break;
        case BG_OP_CROSS_ENTROPY: emit_ce(i, i); break;
        case BG_OP_TRIL: case BG_OP_TRIU: case BG_OP_FLIP: case BG_OP_CONCAT: case BG_OP_CUMSUM:
        case BG_OP_SORT_INDICES: case BG_OP_TOPK_INDICES: emit_shape_op(i, i); break;
        case BG_OP_SCATTER: emit_scatter(i, i); break;
        case BG_OP_RESHAPE:
          if (!copy_elided_.count(i)) emit_copy(i, copy_src_.at(i), resolve(n.in[0]), i);
          break;
        default: err(BG_ERR_UNSUPPORTED, std::string("opcode ") + op_name(n.op));
      }
    }
  }
  // the root must be an owned dense buffer
  {
    int r = root_;
    int rr = resolve(r);
    const View& rv = view_[rr];
    bool owned = !rv.is_const && rv.slot >= 0 && !cp_->slots[rv.slot].external && rv.contiguous() && rv.off == 0 &&
                 cp_->slots[rv.slot].bytes == nodes_[rr].numel() * dtype_size(nodes_[rr].dtype);
    if (!owned) {
      if (rv.is_const) emit_const_fill(rr, nn);
      else {
        // copy through a synthetic RESHAPE-like node
        Node c = nodes_[rr];
        c.op = BG_OP_RESHAPE;
        c.in = {rr};
        nodes_.push_back(c);
        kind_.push_back(K_OTHER);
        View ov;
        ov.set_dense(c.shape, c.rank);
        ov.dtype = c.dtype;
        ov.slot = new_slot(c.numel() * dtype_size(c.dtype), false, (int)nodes_.size() - 1);
        view_.push_back(ov);
        leaflike_.push_back(0);
        const int id = (int)nodes_.size() - 1;
        const View srcv = rv;
        emit_copy(id, srcv, rr, nn);
        rr = id;
      }
      root_ = rr;
    } else {
      root_ = rr;
    }
  }
  return true;
}

void Compiler::schedule() {
  const int nu = (int)punits_.size();
  // node -> producing unit
  std::map<int, int> prod;
  for (int u = 0; u < nu; ++u)
    for (int n : punits_[u].out_nodes) prod[n] = u;
  auto storage_unit = [&](int n) -> int {
    // follow views down to the node that owns the storage
    int guard = 0;
    while (guard++ < 100000) {
      n = resolve(n);
      auto it = prod.find(n);
      if (it != prod.end()) return it->second;
      if (kind_[n] == K_VIEW) { n = nodes_[n].in[0]; continue; }
      return -1;
    }
    return -1;
  };
  std::vector<std::set<int>> deps(nu);
  std::vector<std::vector<int>> users(nu);
  for (int u = 0; u < nu; ++u) {
    for (int n : punits_[u].dep_nodes) {
      int p = storage_unit(n);
      if (p >= 0 && p != u && deps[u].insert(p).second) users[p].push_back(u);
    }
    for (int p : punits_[u].dep_punits)
      if (p >= 0 && p != u && deps[u].insert(p).second) users[p].push_back(u);
  }
  std::vector<int> indeg(nu);
  std::set<std::pair<int, int>> ready;
  for (int u = 0; u < nu; ++u) {
    indeg[u] = (int)deps[u].size();
    if (!indeg[u]) ready.insert({punits_[u].order_key, u});
  }
  std::vector<int> order;
  while (!ready.empty()) {
    auto it = ready.begin();
    int u = it->second;
    ready.erase(it);
    order.push_back(u);
    for (int v : users[u])
      if (--indeg[v] == 0) ready.insert({punits_[v].order_key, v});
  }
  if ((int)order.size() != nu) err(BG_ERR_INVALID, "plan has a dependency cycle between fusion groups");
  // slots read / written per unit, lifetimes
  for (int pos = 0; pos < nu; ++pos) {
    PUnit& pu = punits_[order[pos]];
    Unit u = pu.u;
    for (int n : pu.dep_nodes) {
      int s = view_[resolve(n)].slot;
      if (s >= 0) u.reads.push_back(s);
    }
    for (int n : pu.out_nodes) {
      int s = view_[n].slot;
      if (s >= 0) u.writes.push_back(s);
    }
    for (int s : u.reads) {
      Slot& sl = cp_->slots[s];
      sl.last_unit = pos;
    }
    for (int s : u.writes) {
      Slot& sl = cp_->slots[s];
      if (sl.first_unit < 0) sl.first_unit = pos;
      sl.last_unit = std::max(sl.last_unit, pos);
    }
    cp_->units.push_back(std::move(u));
  }
  const View& rv = view_[root_];
  cp_->root_slot = rv.slot;
  cp_->root_dtype = nodes_[root_].dtype;
  cp_->root_rank = nodes_[root_].rank;
  for (int d = 0; d < cp_->root_rank; ++d) cp_->root_shape[d] = nodes_[root_].shape[d];
  cp_->root_bytes = nodes_[root_].numel() * dtype_size(nodes_[root_].dtype);
  cp_->slots[cp_->root_slot].last_unit = nu;  // survives the plan
  // logical peak over the schedule
  int64_t live = 0, peak = 0;
  for (auto& s : cp_->slots)
    if (s.external) live += s.bytes;
  peak = live;
  for (int pos = 0; pos <= nu; ++pos) {
    for (auto& s : cp_->slots)
      if (!s.external && s.first_unit == pos) live += s.bytes;
    peak = std::max(peak, live);
    for (auto& s : cp_->slots)
      if (!s.external && s.last_unit == pos && s.first_unit >= 0) live -= s.bytes;
  }
  cp_->plan_peak = peak;
  std::ostringstream tr;
  for (auto& u : cp_->units) tr << u.name << "\n";
  cp_->trace = tr.str();
}

std::shared_ptr<CompiledPlan> Compiler::compile() {
  for (int attempt = 0; attempt < 64; ++attempt) {
    if (try_lower()) {
      schedule();
      return cp_;
    }
  }
  err(BG_ERR_UNSUPPORTED, "plan could not be split into launchable fusion groups");
}

}  // namespace

// Reads (and clears) the status word as last copied to the host; call after a synchronisation of the stream, or
// without one to pick up what an earlier copy already delivered.
int take_device_status(bg_context* ctx) {
  ctx->status_pending = false;
  const int st = *ctx->h_status;
  if (st != 0) {
    *ctx->h_status = 0;
    cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream);
  }
  return st;
}

std::string device_status_message(int status_rc) {
  return status_rc == BG_ERR_INDEX_RANGE ? "run_tensor_plan: gather / scatter / cross_entropy index outside its axis, or scatter indices naming one destination twice"
         : status_rc == BG_ERR_DEVICE_TIMEOUT ? "run_tensor_plan: a device-side wait of a tensor-core kernel gave up (status 6)"
                                              : "run_tensor_plan: device-side status " + std::to_string(status_rc);
}

int run_plan(bg_context* ctx, const bg_plan* plan, const bg_plan_input* inputs, int n_inputs, void* out_host,
             size_t out_nbytes, bg_handle* out_handle) {
  if (!plan->steps || plan->n_steps <= 0) return fail(ctx, BG_ERR_INVALID, "run_tensor_plan: empty plan");
  if (n_inputs > 0 && !inputs) return fail(ctx, BG_ERR_INVALID, "run_tensor_plan: null inputs");
  cudaSetDevice(ctx->device);
  // a device-side wait that gave up in an earlier plan whose root stayed on the device is reported here at the latest
  if (ctx->status_pending && *ctx->h_status != 0) {
    const int st = take_device_status(ctx);
    return fail(ctx, st, device_status_message(st) + " (in an earlier plan)");
  }
  uint64_t h = 1469598103934665603ull;
  h = fnv1a(plan->steps, sizeof(bg_plan_step) * (size_t)plan->n_steps, h);
  if (plan->n_ext > 0) h = fnv1a(plan->ext, sizeof(int32_t) * (size_t)plan->n_ext, h);
  h = fnv1a(&plan->root_id, sizeof(int32_t), h);
  const size_t step_bytes = sizeof(bg_plan_step) * (size_t)plan->n_steps;
  const size_t ext_bytes = plan->n_ext > 0 ? sizeof(int32_t) * (size_t)plan->n_ext : 0;
  auto same_bytes = [&](const CompiledPlan& c) {
    if (c.key_bytes.size() != step_bytes + ext_bytes + sizeof(int32_t)) return false;
    const unsigned char* k = c.key_bytes.data();
    return memcmp(k, plan->steps, step_bytes) == 0 && (ext_bytes == 0 || memcmp(k + step_bytes, plan->ext, ext_bytes) == 0) &&
           memcmp(k + step_bytes + ext_bytes, &plan->root_id, sizeof(int32_t)) == 0;
  };
  std::shared_ptr<CompiledPlan> cp;
  auto it = ctx->plan_cache.find(h);
  if (it != ctx->plan_cache.end() && same_bytes(*it->second)) {
    cp = it->second;
    ctx->cache_hits++;
  } else {
    try {
      Compiler c(ctx, plan);
      cp = c.compile();
    } catch (CompileError& ce) {
      return fail(ctx, ce.code > 0 ? ce.code : BG_ERR_UNSUPPORTED, "run_tensor_plan: " + ce.msg);
    }
    cp->key_bytes.resize(step_bytes + ext_bytes + sizeof(int32_t));
    memcpy(cp->key_bytes.data(), plan->steps, step_bytes);
    if (ext_bytes) memcpy(cp->key_bytes.data() + step_bytes, plan->ext, ext_bytes);
    memcpy(cp->key_bytes.data() + step_bytes + ext_bytes, &plan->root_id, sizeof(int32_t));
    if (ctx->plan_cache.size() > 256) ctx->plan_cache.clear();
    ctx->plan_cache[h] = cp;     // a different plan with the same hash replaces the old entry
    ctx->cache_misses++;
  }
  ctx->last_trace = cp->trace;
  if (out_host && (int64_t)out_nbytes != cp->root_bytes)
    return fail(ctx, BG_ERR_INVALID, "run_tensor_plan: destination holds " + std::to_string(out_nbytes) + " bytes, the root has " +
                                         std::to_string(cp->root_bytes));
  Run run;
  run.ctx = ctx;
  run.ptr.assign(cp->slots.size(), nullptr);
  run.from_handle.assign(cp->slots.size(), 0);
  std::vector<std::pair<void*, int64_t>> temp_uploads;
  std::vector<int> allocated;  // slots allocated by this run
  auto cleanup = [&](bool keep_root) {
    for (int s : allocated) {
      if (keep_root && s == cp->root_slot) continue;
      if (run.ptr[s]) dev_free(ctx, run.ptr[s], cp->slots[s].bytes);
      run.ptr[s] = nullptr;
    }
    allocated.clear();
    for (auto& t : temp_uploads) dev_free(ctx, t.first, t.second);
    temp_uploads.clear();
  };
  // bind BUFFER steps
  for (size_t b = 0; b < cp->buffers.size(); ++b) {
    const int vid = cp->buffers[b].first, slot = cp->buffers[b].second;
    const bg_plan_input* found = nullptr;
    for (int i = 0; i < n_inputs; ++i)
      if (inputs[i].value_id == vid) { found = &inputs[i]; break; }
    if (!found) { cleanup(false); return fail(ctx, BG_ERR_INVALID, "run_tensor_plan: no input bound to BUFFER value_id " + std::to_string(vid)); }
    const int64_t want = cp->buffer_bytes[b];
    if (found->handle != 0) {
      auto hit = ctx->handles.find(found->handle);
      if (hit == ctx->handles.end()) { cleanup(false); return fail(ctx, BG_ERR_UNKNOWN_HANDLE, "run_tensor_plan: unknown handle " + std::to_string(found->handle)); }
      if (hit->second.bytes != want) { cleanup(false); return fail(ctx, BG_ERR_INVALID, "run_tensor_plan: handle for value_id " + std::to_string(vid) + " holds " + std::to_string(hit->second.bytes) + " bytes, the plan declares " + std::to_string(want)); }
      run.ptr[slot] = hit->second.ptr;
      run.from_handle[slot] = 1;
    } else {
      if ((int64_t)found->nbytes != want || (want > 0 && !found->data)) { cleanup(false); return fail(ctx, BG_ERR_INVALID, "run_tensor_plan: data for value_id " + std::to_string(vid) + " has " + std::to_string(found->nbytes) + " bytes, the plan declares " + std::to_string(want)); }
      void* p = nullptr;
      if (int rc = dev_alloc(ctx, want, &p)) { cleanup(false); return rc; }
      temp_uploads.push_back({p, want});
      if (int rc = h2d(ctx, p, found->data, (size_t)want)) { cleanup(false); return rc; }
      run.ptr[slot] = p;
    }
  }
  // execute
  const int nu = (int)cp->units.size();
  for (int pos = 0; pos < nu; ++pos) {
    Unit& u = cp->units[pos];
    for (int s : u.writes)
      if (!run.ptr[s]) {
        if (int rc = dev_alloc(ctx, cp->slots[s].bytes, &run.ptr[s])) { cleanup(false); return rc; }
        allocated.push_back(s);
      }
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (ctx->profiling) {
      cudaEventCreate(&e0);
      cudaEventCreate(&e1);
      cudaEventRecord(e0, ctx->stream);
    }
    int rc = u.fn(run);
    if (ctx->profiling) {
      cudaEventRecord(e1, ctx->stream);
      ctx->pending_events.push_back({u.name, {e0, e1}});
    }
    if (rc) { cleanup(false); return rc; }
    ctx->launches += u.launches;
    // free intermediates whose last reader this was
    for (size_t k = 0; k < allocated.size();) {
      int s = allocated[k];
      if (cp->slots[s].last_unit == pos && s != cp->root_slot) {
        dev_free(ctx, run.ptr[s], cp->slots[s].bytes);
        run.ptr[s] = nullptr;
        allocated[k] = allocated.back();
        allocated.pop_back();
      } else ++k;
    }
  }
  if (cp->plan_peak > ctx->plan_peak) ctx->plan_peak = cp->plan_peak;
  if (!run.ptr[cp->root_slot]) { cleanup(false); return fail(ctx, BG_ERR_INVALID, "run_tensor_plan: root was not produced"); }
  int status_rc = BG_OK;
  if (cp->uses_status || cp->uses_wait_status)
    cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream);
  if ((cp->uses_status || cp->uses_wait_status) && out_host) {
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) { cleanup(false); return cuda_fail(ctx, e, "plan execution"); }
    status_rc = take_device_status(ctx);
  } else if (cp->uses_status || cp->uses_wait_status) {
    ctx->status_pending = true;
  }
  if (status_rc) {
    cleanup(false);
    return fail(ctx, status_rc, device_status_message(status_rc));
  }
  if (out_host) {
    int rc = d2h(ctx, out_host, run.ptr[cp->root_slot], (size_t)cp->root_bytes);
    cleanup(false);
    return rc;
  }
  *out_handle = mint_handle(ctx, run.ptr[cp->root_slot], cp->root_bytes, cp->root_dtype, cp->root_shape, cp->root_rank);
  cleanup(true);
  return BG_OK;
}

}  // namespace bg

extern "C" int bg_compile_plan_dry(const bg_plan* plan, int fusion, char* out, size_t capacity) {
  // Host-only: compiles the plan into its launch list without touching a device.
  if (!plan || !out || capacity == 0) return BG_ERR_INVALID;
  bg_context fake;
  fake.fusion = (fusion & 1) != 0;
  fake.sm_count = 148;
  bg::g_tc_assume_available = (fusion & 2) != 0;   // lower as on a B200 (tensor-core kernels selectable)
  std::string text;
  int rc = BG_OK;
  try {
    bg::Compiler c(&fake, plan);
    auto cp = c.compile();
    text = cp->trace;
  } catch (bg::CompileError& ce) {
    text = "error: " + ce.msg;
    rc = ce.code > 0 ? ce.code : BG_ERR_UNSUPPORTED;
  }
  bg::g_tc_assume_available = false;
  strncpy(out, text.c_str(), capacity - 1);
  out[capacity - 1] = 0;
  return rc;
}

