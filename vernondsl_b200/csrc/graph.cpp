// Execution graph: a small tensor graph whose elementwise chains are fused into single map
// kernels, with reverse-mode differentiation and kernel selection.  Host code only; every kernel
// it plans is launched through the operator registry of this library.
//
// The reference project has no execution graph or autodiff; this layer exists so that a caller
// states a computation once (as fractal.py states a kernel body) and the library decides which
// hand-written kernels run it.
//
// Shapes: FULL [rows][cols], ROWVEC [cols] (broadcast down the rows), COLVEC [rows] (one value per
// row), SCALAR.  Elementwise nodes take the join of their operands' shapes.
//
// Planning rules
//   * Results that must exist in memory ("roots"): graph outputs and operands of reductions and
//     softmax.  Inputs, reduction results and softmax results are "leaves" (read from memory).
//   * stage(root) = 1 + max stage of the leaves it reaches through elementwise nodes; a reduction's
//     stage is 1 + its operand's.  Roots with the same shape and stage that share a leaf or an
//     interior node are merged into ONE kernel with several outputs (limits: 8 inputs, 4 outputs,
//     64 instructions).  Steps run in stage order, which respects every dependency.
//   * A fused group that is exactly the map-workload chain runs the specialised `fused_map`
//     kernel; a graph whose outputs are the tanh-MSE loss and/or its three gradients runs the
//     hand-fused `mse_tanh_bwd` / `mse_tanh_fwd` kernels.  Everything else runs `map_tape`.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <set>
#include <sstream>
#include <string>
#include <vector>

#include "vrhi_internal.h"

using namespace vrhi;

namespace {

enum Kind { K_INPUT, K_CONST, K_UNARY, K_BINARY, K_EXPAND, K_REDUCE, K_SOFTMAX };

struct Node {
  Kind kind;
  int op = 0;
  int a = -1, b = -1;
  float imm = 0.f;
  int shape = VRHI_SHAPE_FULL;
  vrhi_buffer buf = nullptr;
};

struct Step {
  int stage = 0;
  int order = 0;
  int op = -1;  // registry id
  std::vector<vrhi_arg> args;
  std::vector<unsigned char> params;
  std::string text;
};

int join_shape(int a, int b) {
  if (a == b) return a;
  if (a == VRHI_SHAPE_SCALAR) return b;
  if (b == VRHI_SHAPE_SCALAR) return a;
  return VRHI_SHAPE_FULL;  // FULL with anything, or ROWVEC with COLVEC
}

bool shape_le(int small, int big) { return join_shape(small, big) == big; }

const char *shape_name(int s) {
  static const char *n[] = {"full", "rowvec", "colvec", "scalar"};
  return n[s & 3];
}

bool is_elementwise(Kind k) { return k == K_CONST || k == K_UNARY || k == K_BINARY || k == K_EXPAND; }

bool commutative(int op) { return op == VRHI_T_ADD || op == VRHI_T_MUL || op == VRHI_T_MAX || op == VRHI_T_MIN || op == VRHI_T_EQ; }

const char *kTapeNames[] = {"const", "add", "sub", "mul", "div", "max", "min", "fma", "neg", "abs", "square", "sqrt",
                            "rsqrt", "recip", "exp", "log", "tanh", "sigmoid", "relu", "cos", "sin", "sign", "step", "eq"};

}  // namespace

struct vrhi_graph_t {
  vrhi_device_t *dev;
  uint64_t rows, cols;
  std::vector<Node> nodes;
  std::vector<std::pair<int, vrhi_buffer>> outputs;
  struct GradRec { int loss, wrt, node; };
  std::vector<GradRec> grads;
  std::vector<Step> steps;
  std::vector<vrhi_buffer> temps;
  bool compiled = false;
  uint32_t flags = 0;
  std::string plan;

  uint64_t elems(int shape) const {
    switch (shape) {
      case VRHI_SHAPE_FULL: return rows * cols;
      case VRHI_SHAPE_ROWVEC: return cols;
      case VRHI_SHAPE_COLVEC: return rows;
      default: return 1;
    }
  }
  int add(const Node &n) {
    nodes.push_back(n);
    compiled = false;
    return (int)nodes.size() - 1;
  }
  bool valid(int id) const { return id >= 0 && id < (int)nodes.size(); }
};

namespace {

typedef vrhi_graph_t G;

// ------------------------------------------------------------------ node construction -------
int mk_const(G *g, float v) {
  Node n; n.kind = K_CONST; n.op = VRHI_T_CONST; n.imm = v; n.shape = VRHI_SHAPE_SCALAR;
  return g->add(n);
}
int mk_unary(G *g, int op, int a) {
  Node n; n.kind = K_UNARY; n.op = op; n.a = a; n.shape = g->nodes[a].shape;
  return g->add(n);
}
int mk_binary(G *g, int op, int a, int b) {
  Node n; n.kind = K_BINARY; n.op = op; n.a = a; n.b = b;
  n.shape = join_shape(g->nodes[a].shape, g->nodes[b].shape);
  return g->add(n);
}
int mk_expand(G *g, int a, int shape) {
  if (g->nodes[a].shape == shape) return a;
  Node n; n.kind = K_EXPAND; n.a = a; n.shape = shape;
  return g->add(n);
}
int reduce_shape(int op, int in_shape) {
  switch (op) {
    case VRHI_R_ROW_SUM: case VRHI_R_ROW_MAX: return in_shape == VRHI_SHAPE_FULL ? VRHI_SHAPE_COLVEC : -1;
    case VRHI_R_COL_SUM: return in_shape == VRHI_SHAPE_FULL ? VRHI_SHAPE_ROWVEC : -1;
    case VRHI_R_SUM_ALL: case VRHI_R_MEAN_ALL: return in_shape == VRHI_SHAPE_SCALAR ? -1 : VRHI_SHAPE_SCALAR;
    default: return -1;
  }
}
int mk_reduce(G *g, int op, int a) {
  Node n; n.kind = K_REDUCE; n.op = op; n.a = a; n.shape = reduce_shape(op, g->nodes[a].shape);
  return g->add(n);
}

// ------------------------------------------------------------------ differentiation ---------
struct Autodiff {
  G *g;
  std::vector<int> adj;  // node -> adjoint node, -1 if none yet

  // Bring `c`, the adjoint of a value of shape `out_shape`, down to an operand of shape `to`.
  int unbroadcast(int c, int out_shape, int to) {
    if (to == out_shape) return c;  // no broadcast happened for this operand
    int full = mk_expand(g, c, out_shape);  // the sum below must see every broadcast copy
    if (out_shape == VRHI_SHAPE_FULL) {
      if (to == VRHI_SHAPE_ROWVEC) return mk_reduce(g, VRHI_R_COL_SUM, full);
      if (to == VRHI_SHAPE_COLVEC) return mk_reduce(g, VRHI_R_ROW_SUM, full);
    }
    return mk_reduce(g, VRHI_R_SUM_ALL, full);  // to == SCALAR
  }
  void accumulate(int node, int c) {
    if (g->nodes[node].kind == K_CONST) return;
    adj[node] = adj[node] < 0 ? c : mk_binary(g, VRHI_T_ADD, adj[node], c);
  }
  void to_operand(int operand, int c, int out_shape) {
    if (g->nodes[operand].kind == K_CONST) return;
    accumulate(operand, unbroadcast(c, out_shape, g->nodes[operand].shape));
  }

  int run(int loss, const int *wrt, int n_wrt, int *out) {
    const int n0 = (int)g->nodes.size();
    adj.assign(n0, -1);
    std::vector<char> needed(n0, 0);
    needed[loss] = 1;
    for (int i = loss; i >= 0; --i) {
      if (!needed[i]) continue;
      if (g->nodes[i].a >= 0) needed[g->nodes[i].a] = 1;
      if (g->nodes[i].b >= 0) needed[g->nodes[i].b] = 1;
    }
    adj[loss] = mk_const(g, 1.0f);
    for (int i = loss; i >= 0; --i) {
      if (!needed[i] || adj[i] < 0) continue;
      const Node n = g->nodes[i];  // copy: the vector grows below
      const int gi = adj[i];
      const int S = n.shape;
      switch (n.kind) {
        case K_INPUT: case K_CONST: break;
        case K_EXPAND: to_operand(n.a, gi, S); break;
        case K_BINARY: {
          const int a = n.a, b = n.b;
          switch (n.op) {
            case VRHI_T_ADD: to_operand(a, gi, S); to_operand(b, gi, S); break;
            case VRHI_T_SUB: to_operand(a, gi, S); to_operand(b, mk_unary(g, VRHI_T_NEG, gi), S); break;
            case VRHI_T_MUL:
              to_operand(a, mk_binary(g, VRHI_T_MUL, gi, b), S);
              to_operand(b, mk_binary(g, VRHI_T_MUL, gi, a), S);
              break;
            case VRHI_T_DIV: {
              int q = mk_binary(g, VRHI_T_DIV, gi, b);
              to_operand(a, q, S);
              to_operand(b, mk_unary(g, VRHI_T_NEG, mk_binary(g, VRHI_T_MUL, q, i)), S);
              break;
            }
            case VRHI_T_MAX: case VRHI_T_MIN: {
              // derivative flows to the operand that was selected (to `a` on ties)
              int d = n.op == VRHI_T_MAX ? mk_binary(g, VRHI_T_SUB, b, a) : mk_binary(g, VRHI_T_SUB, a, b);
              int to_b = mk_unary(g, VRHI_T_STEP, d);
              int to_a = mk_binary(g, VRHI_T_SUB, mk_const(g, 1.0f), to_b);
              to_operand(a, mk_binary(g, VRHI_T_MUL, gi, to_a), S);
              to_operand(b, mk_binary(g, VRHI_T_MUL, gi, to_b), S);
              break;
            }
            case VRHI_T_EQ: break;  // piecewise constant
            default: return fail(VRHI_ERR_GRAPH, "grad: binary op %d is not differentiable here", n.op);
          }
          break;
        }
        case K_UNARY: {
          const int a = n.a;
          int d = -1;  // d(out)/d(a)
          switch (n.op) {
            case VRHI_T_NEG: d = mk_const(g, -1.0f); break;
            case VRHI_T_ABS: d = mk_unary(g, VRHI_T_SIGN, a); break;
            case VRHI_T_SQUARE: d = mk_binary(g, VRHI_T_MUL, mk_const(g, 2.0f), a); break;
            case VRHI_T_SQRT: d = mk_binary(g, VRHI_T_DIV, mk_const(g, 0.5f), i); break;
            case VRHI_T_RSQRT: d = mk_binary(g, VRHI_T_MUL, mk_const(g, -0.5f), mk_binary(g, VRHI_T_DIV, i, a)); break;
            case VRHI_T_RECIP: d = mk_unary(g, VRHI_T_NEG, mk_unary(g, VRHI_T_SQUARE, i)); break;
            case VRHI_T_EXP: d = i; break;
            case VRHI_T_LOG: d = mk_unary(g, VRHI_T_RECIP, a); break;
            case VRHI_T_TANH: d = mk_binary(g, VRHI_T_SUB, mk_const(g, 1.0f), mk_unary(g, VRHI_T_SQUARE, i)); break;
            case VRHI_T_SIGMOID: d = mk_binary(g, VRHI_T_MUL, i, mk_binary(g, VRHI_T_SUB, mk_const(g, 1.0f), i)); break;
            case VRHI_T_RELU: d = mk_unary(g, VRHI_T_STEP, a); break;
            case VRHI_T_COS: d = mk_unary(g, VRHI_T_NEG, mk_unary(g, VRHI_T_SIN, a)); break;
            case VRHI_T_SIN: d = mk_unary(g, VRHI_T_COS, a); break;
            case VRHI_T_SIGN: case VRHI_T_STEP: d = -2; break;
            default: return fail(VRHI_ERR_GRAPH, "grad: unary op %d is not differentiable here", n.op);
          }
          if (d >= 0) to_operand(a, mk_binary(g, VRHI_T_MUL, gi, d), S);
          break;
        }
        case K_REDUCE: {
          const int a = n.a;
          const int as = g->nodes[a].shape;
          switch (n.op) {
            case VRHI_R_ROW_SUM: case VRHI_R_COL_SUM: case VRHI_R_SUM_ALL:
              accumulate(a, gi);  // every summand sees the adjoint unchanged (broadcast is implicit)
              break;
            case VRHI_R_MEAN_ALL:
              accumulate(a, mk_binary(g, VRHI_T_MUL, gi, mk_const(g, (float)(1.0 / (double)g->elems(as)))));
              break;
            case VRHI_R_ROW_MAX:
              accumulate(a, mk_binary(g, VRHI_T_MUL, gi, mk_binary(g, VRHI_T_EQ, a, i)));
              break;
            default: return fail(VRHI_ERR_GRAPH, "grad: reduction %d is not differentiable here", n.op);
          }
          break;
        }
        case K_SOFTMAX: {
          // d a = out * (g - rowsum(g * out))
          int go = mk_expand(g, mk_binary(g, VRHI_T_MUL, gi, i), VRHI_SHAPE_FULL);
          int rs = mk_reduce(g, VRHI_R_ROW_SUM, go);
          accumulate(n.a, mk_binary(g, VRHI_T_MUL, i, mk_binary(g, VRHI_T_SUB, gi, rs)));
          break;
        }
      }
    }
    for (int k = 0; k < n_wrt; ++k) {
      int w = wrt[k];
      int r = adj[w] >= 0 ? adj[w] : mk_const(g, 0.0f);
      r = mk_expand(g, r, g->nodes[w].shape);
      out[k] = r;
      g->grads.push_back({loss, w, r});
    }
    return VRHI_OK;
  }
};

// ------------------------------------------------------------------ planning ----------------
struct Planner {
  G *g;
  std::vector<char> live, root;
  std::vector<int> stage;
  std::vector<vrhi_buffer> storage;  // node -> buffer holding it (leaves and roots)
  std::map<int, int> op_ids;
  // Elementwise roots that are summed over the rows inside the map kernel instead of being stored:
  // root -> the [cols] array that receives the sums.  `folded_nodes`: column-sum nodes that need no
  // step of their own; `folded_mid`: full sums / means whose first half (the column sum) is done.
  std::map<int, vrhi_buffer> folded;
  std::set<int> folded_nodes;
  std::map<int, vrhi_buffer> folded_mid;
  int next_order = 0;

  bool leaf(int i) const {
    Kind k = g->nodes[i].kind;
    return k == K_INPUT || k == K_REDUCE || k == K_SOFTMAX;
  }

  int op_id(const char *name, int *out) {
    return vrhi_op_lookup(name, out);
  }

  int node_stage(int i) {
    if (stage[i] >= 0) return stage[i];
    const Node &n = g->nodes[i];
    int s = 0;
    if (n.kind == K_INPUT || n.kind == K_CONST) s = 0;
    else if (n.kind == K_REDUCE || n.kind == K_SOFTMAX) s = node_stage(n.a) + 1;
    else {
      // elementwise: stage of the kernel that would compute it = 1 + max over reached leaves
      int m = 0;
      if (n.a >= 0) m = std::max(m, leaf(n.a) ? node_stage(n.a) + 1 : node_stage(n.a));
      if (n.b >= 0) m = std::max(m, leaf(n.b) ? node_stage(n.b) + 1 : node_stage(n.b));
      s = m;
    }
    return stage[i] = s;
  }

  // Collect the leaves and interior nodes of the expression rooted at r.
  void collect(int i, std::set<int> &leaves, std::set<int> &interior) {
    if (leaf(i)) { leaves.insert(i); return; }
    if (!interior.insert(i).second) return;
    const Node &n = g->nodes[i];
    if (n.a >= 0) collect(n.a, leaves, interior);
    if (n.b >= 0) collect(n.b, leaves, interior);
  }

  int temp_for(int node) {
    vrhi_buffer b = nullptr;
    VRHI_TRY(vrhi_buffer_create(g->dev, g->elems(g->nodes[node].shape) * 4, VRHI_STORAGE_BUFFER, &b));
    g->temps.push_back(b);
    storage[node] = b;
    return VRHI_OK;
  }

  vrhi_arg arg_of(int node, int cls) {
    vrhi_arg a{};
    a.buffer = storage[node];
    a.offset = 0;
    a.bytes = g->elems(g->nodes[node].shape) * 4;
    a.arg_class = cls;
    return a;
  }

  // Emit one map kernel computing `roots` (same shape, same stage).
  int emit_map(const std::vector<int> &roots, const std::set<int> &leaves, int st) {
    const int shape = g->nodes[roots[0]].shape;
    vrhi_tape_params P{};
    P.size = sizeof P;
    std::map<int, int> leaf_index;
    std::vector<int> leaf_list(leaves.begin(), leaves.end());
    if (leaf_list.size() > VRHI_TAPE_MAX_INPUTS) return fail(VRHI_ERR_GRAPH, "a fused group reads %zu arrays; the limit is %d", leaf_list.size(), VRHI_TAPE_MAX_INPUTS);
    for (size_t k = 0; k < leaf_list.size(); ++k) {
      leaf_index[leaf_list[k]] = (int)k;
      const int ls = g->nodes[leaf_list[k]].shape;
      if (!shape_le(ls, shape)) return fail(VRHI_ERR_GRAPH, "internal: leaf shape %s does not broadcast to %s", shape_name(ls), shape_name(shape));
      if (ls != shape) {
        if (ls == VRHI_SHAPE_ROWVEC) P.row_vector_mask |= 1u << k;
        else if (ls == VRHI_SHAPE_COLVEC) P.col_vector_mask |= 1u << k;
        else P.scalar_mask |= 1u << k;
      }
    }
    P.n_inputs = (uint32_t)leaf_list.size();
    P.n_outputs = (uint32_t)roots.size();
    switch (shape) {
      case VRHI_SHAPE_FULL: P.rows = g->rows; P.cols = g->cols; break;
      case VRHI_SHAPE_ROWVEC: P.rows = 1; P.cols = g->cols; break;
      case VRHI_SHAPE_COLVEC: P.rows = g->rows; P.cols = 1; break;
      default: P.rows = 1; P.cols = 1; break;
    }
    std::map<int, int> value_of;  // node -> tape value index
    int rc = VRHI_OK;
    // iterative post-order would be overkill for 64 instructions: recursion depth is bounded by it
    struct Rec {
      Planner *pl; vrhi_tape_params &P; std::map<int, int> &value_of; std::map<int, int> &leaf_index; int &rc;
      int go(int i) {
        if (pl->leaf(i)) return leaf_index.at(i);
        auto it = value_of.find(i);
        if (it != value_of.end()) return it->second;
        const Node &n = pl->g->nodes[i];
        int v;
        if (n.kind == K_EXPAND) {
          v = go(n.a);
        } else {
          int va = n.a >= 0 ? go(n.a) : 0, vb = n.b >= 0 ? go(n.b) : 0;
          if (rc != VRHI_OK) return 0;
          if (P.n_instr >= VRHI_TAPE_MAX_INSTR) { rc = fail(VRHI_ERR_GRAPH, "a fused group needs more than %d instructions", VRHI_TAPE_MAX_INSTR); return 0; }
          vrhi_tape_instr &I = P.instr[P.n_instr];
          I.op = (uint16_t)n.op; I.a = (uint16_t)va; I.b = (uint16_t)vb; I.c = 0; I.imm = n.imm;
          v = (int)(P.n_inputs + P.n_instr);
          ++P.n_instr;
        }
        value_of[i] = v;
        return v;
      }
    } rec{this, P, value_of, leaf_index, rc};
    for (size_t k = 0; k < roots.size(); ++k) {
      int v = rec.go(roots[k]);
      if (rc != VRHI_OK) return rc;
      if (v < (int)P.n_inputs) {
        // the root is a bare (possibly broadcast) leaf: copy through an explicit add-zero
        if (P.n_instr + 2 > VRHI_TAPE_MAX_INSTR) return fail(VRHI_ERR_GRAPH, "a fused group needs more than %d instructions", VRHI_TAPE_MAX_INSTR);
        vrhi_tape_instr &Z = P.instr[P.n_instr];
        Z.op = VRHI_T_CONST; Z.imm = 0.f;
        int zv = (int)(P.n_inputs + P.n_instr++);
        vrhi_tape_instr &A = P.instr[P.n_instr];
        A.op = VRHI_T_ADD; A.a = (uint16_t)v; A.b = (uint16_t)zv;
        v = (int)(P.n_inputs + P.n_instr++);
      }
      P.out_value[k] = (uint32_t)v;
    }
    Step s;
    s.stage = st;
    s.order = next_order++;
    for (int l : leaf_list) s.args.push_back(arg_of(l, VRHI_INPUT));
    for (size_t k = 0; k < roots.size(); ++k) {
      auto f = folded.find(roots[k]);
      if (f == folded.end()) {
        s.args.push_back(arg_of(roots[k], VRHI_OUTPUT));
      } else {  // the map kernel writes the column sums straight into the reduction's array
        P.colsum_mask |= 1u << k;
        vrhi_arg a{};
        a.buffer = f->second; a.offset = 0; a.bytes = g->cols * 4; a.arg_class = VRHI_OUTPUT;
        s.args.push_back(a);
      }
    }
    std::ostringstream text;
    bool special = false;
    if (!(g->flags & 1u) && P.colsum_mask == 0 && shape == VRHI_SHAPE_FULL && roots.size() == 1 && leaf_list.size() == 3 && P.row_vector_mask == 0 && P.col_vector_mask == 0 && P.scalar_mask == 0) {
      // the map-workload chain, operands of commutative nodes in any order
      special = match_chain(roots[0], leaf_list, &s);
    }
    if (special) {
      text << "fused_map   stage " << st << " n=" << g->rows * g->cols << " (specialised chain)";
    } else {
      VRHI_TRY(op_id("map_tape", &s.op));
      s.params.assign((unsigned char *)&P, (unsigned char *)&P + sizeof P);
      text << "map_tape    stage " << st << " shape=" << shape_name(shape) << " inputs=" << P.n_inputs << " outputs=" << P.n_outputs
           << " instr=" << P.n_instr;
      for (uint32_t k = 0; k < P.n_outputs; ++k)
        if ((P.colsum_mask >> k) & 1u) text << " (output " << k << ": col_sum folded into the kernel)";
    }
    s.text = text.str();
    g->steps.push_back(s);
    return VRHI_OK;
  }

  // Structural match of  tanh(a*x + y) * exp(-0.5*x*x) + sqrt(|y| + 1e-3)  (commutative operands in any order).
  bool is_const(int i, float v) const { const Node &n = g->nodes[i]; return n.kind == K_CONST && n.imm == v; }
  int strip(int i) const { while (g->nodes[i].kind == K_EXPAND) i = g->nodes[i].a; return i; }
  bool bin(int i, int op, int *a, int *b) const {
    i = strip(i);
    const Node &n = g->nodes[i];
    if (n.kind != K_BINARY || n.op != op) return false;
    *a = strip(n.a); *b = strip(n.b);
    return true;
  }
  bool un(int i, int op, int *a) const {
    i = strip(i);
    const Node &n = g->nodes[i];
    if (n.kind != K_UNARY || n.op != op) return false;
    *a = strip(n.a);
    return true;
  }
  bool full_input(int i) const { return g->nodes[i].kind == K_INPUT && g->nodes[i].shape == VRHI_SHAPE_FULL; }

  // u = a*x + y with x known: returns a, y
  bool match_axpy(int u, int x, int *a, int *y) const {
    int p, q;
    if (!bin(u, VRHI_T_ADD, &p, &q)) return false;
    for (int sw = 0; sw < 2; ++sw) {
      int m0, m1;
      if (bin(p, VRHI_T_MUL, &m0, &m1) && full_input(q)) {
        if (m1 == x && full_input(m0)) { *a = m0; *y = q; return true; }
        if (m0 == x && full_input(m1)) { *a = m1; *y = q; return true; }
      }
      std::swap(p, q);
    }
    return false;
  }
  // e = exp(-0.5*x*x) in any association; returns x
  bool match_gauss(int e, int *x) const {
    int arg;
    if (!un(e, VRHI_T_EXP, &arg)) return false;
    int p, q;
    if (!bin(arg, VRHI_T_MUL, &p, &q)) return false;
    for (int sw = 0; sw < 2; ++sw) {
      int r, s2;
      // (-0.5*x)*x  or  -0.5*(x*x)  or  -0.5*square(x)
      if (bin(p, VRHI_T_MUL, &r, &s2)) {
        if (is_const(r, -0.5f) && s2 == q && full_input(q)) { *x = q; return true; }
        if (is_const(s2, -0.5f) && r == q && full_input(q)) { *x = q; return true; }
        if (is_const(q, -0.5f) && r == s2 && full_input(r)) { *x = r; return true; }
      }
      int sq;
      if (is_const(q, -0.5f) && un(p, VRHI_T_SQUARE, &sq) && full_input(sq)) { *x = sq; return true; }
      std::swap(p, q);
    }
    return false;
  }
  bool match_chain(int root, const std::vector<int> &leaf_list, Step *s) {
    int p, q;
    if (!bin(root, VRHI_T_ADD, &p, &q)) return false;
    for (int sw = 0; sw < 2; ++sw) {
      // p = tanh(..)*exp(..), q = sqrt(|y| + 1e-3)
      int prod0, prod1, sq_arg;
      if (bin(p, VRHI_T_MUL, &prod0, &prod1) && un(q, VRHI_T_SQRT, &sq_arg)) {
        for (int sw2 = 0; sw2 < 2; ++sw2) {
          int x, u, a, y;
          if (match_gauss(prod1, &x) && un(prod0, VRHI_T_TANH, &u) && match_axpy(u, x, &a, &y)) {
            int s0, s1, ay;
            if (bin(sq_arg, VRHI_T_ADD, &s0, &s1)) {
              for (int sw3 = 0; sw3 < 2; ++sw3) {
                if (is_const(s1, 1e-3f) && un(s0, VRHI_T_ABS, &ay) && ay == y && a != x && a != y && x != y) {
                  if (leaf_list.size() != 3) return false;
                  if (vrhi_op_lookup("fused_map", &s->op) != VRHI_OK) return false;
                  vrhi_arg out = s->args.back();
                  s->args.clear();
                  s->args.push_back(arg_of(a, VRHI_INPUT));
                  s->args.push_back(arg_of(x, VRHI_INPUT));
                  s->args.push_back(arg_of(y, VRHI_INPUT));
                  s->args.push_back(out);
                  vrhi_map_params mp{};
                  mp.size = sizeof mp;
                  mp.n = g->rows * g->cols;
                  s->params.assign((unsigned char *)&mp, (unsigned char *)&mp + sizeof mp);
                  return true;
                }
                std::swap(s0, s1);
              }
            }
          }
          std::swap(prod0, prod1);
        }
      }
      std::swap(p, q);
    }
    return false;
  }

  // loss = mean_all(square(tanh(W*x + b) - t)); returns the four inputs.
  bool match_mse_loss(int loss, int *W, int *x, int *b, int *t) const {
    const Node &L = g->nodes[loss];
    if (L.kind != K_REDUCE || L.op != VRHI_R_MEAN_ALL) return false;
    int d, y, u, p, q;
    if (!un(L.a, VRHI_T_SQUARE, &d)) return false;
    if (!bin(d, VRHI_T_SUB, &y, t)) return false;
    if (!full_input(*t)) return false;
    if (!un(y, VRHI_T_TANH, &u)) return false;
    if (!bin(u, VRHI_T_ADD, &p, &q)) return false;
    for (int sw = 0; sw < 2; ++sw) {
      int m0, m1;
      if (bin(p, VRHI_T_MUL, &m0, &m1) && g->nodes[q].kind == K_INPUT && g->nodes[q].shape == VRHI_SHAPE_ROWVEC && full_input(m0) && full_input(m1)) {
        *W = m0; *x = m1; *b = q;
        return true;
      }
      std::swap(p, q);
    }
    return false;
  }

  // Whole-graph selection of the hand-fused loss / gradient kernels.
  int try_mse(bool *done) {
    *done = false;
    if (g->flags & 1u) return VRHI_OK;
    if (g->outputs.empty()) return VRHI_OK;
    int loss = -1;
    for (auto &o : g->outputs) {
      bool found = false;
      for (auto &gr : g->grads)
        if (gr.node == o.first) { if (loss >= 0 && loss != gr.loss) return VRHI_OK; loss = gr.loss; found = true; }
      if (!found) { if (loss >= 0 && loss != o.first) return VRHI_OK; loss = o.first; }
    }
    int W, x, b, t;
    if (loss < 0 || !match_mse_loss(loss, &W, &x, &b, &t)) return VRHI_OK;
    if (W == x || W == t || x == t) return VRHI_OK;
    vrhi_buffer oW = nullptr, ox = nullptr, ob = nullptr, oL = nullptr;
    bool any_grad = false;
    for (auto &o : g->outputs) {
      if (o.first == loss) { if (oL) return VRHI_OK; oL = o.second; continue; }
      int wrt = -1;
      for (auto &gr : g->grads) if (gr.node == o.first) wrt = gr.wrt;
      // W*x is symmetric: the gradient with respect to either factor is g times the other one
      if (wrt == W) { if (oW) return VRHI_OK; oW = o.second; }
      else if (wrt == x) { if (ox) return VRHI_OK; ox = o.second; }
      else if (wrt == b) { if (ob) return VRHI_OK; ob = o.second; }
      else return VRHI_OK;
      any_grad = true;
    }
    Step s;
    s.stage = 1;
    s.order = next_order++;
    vrhi_mse_params mp{};
    mp.size = sizeof mp;
    mp.rows = g->rows; mp.cols = g->cols; mp.denom = 0.0;
    s.params.assign((unsigned char *)&mp, (unsigned char *)&mp + sizeof mp);
    auto in_arg = [&](int node) { vrhi_arg a{}; a.buffer = g->nodes[node].buf; a.bytes = g->elems(g->nodes[node].shape) * 4; a.arg_class = VRHI_INPUT; return a; };
    auto out_arg = [&](vrhi_buffer bf, uint64_t bytes) { vrhi_arg a{}; a.buffer = bf; a.bytes = bytes; a.arg_class = VRHI_OUTPUT; return a; };
    s.args = {in_arg(W), in_arg(x), in_arg(b), in_arg(t)};
    const uint64_t full = g->rows * g->cols * 4;
    if (any_grad) {
      VRHI_TRY(vrhi_op_lookup("mse_tanh_bwd", &s.op));
      vrhi_buffer *slots[3] = {&oW, &ox, &ob};
      const uint64_t sizes[3] = {full, full, g->cols * 4};
      for (int k = 0; k < 3; ++k)
        if (!*slots[k]) {  // a gradient nobody asked for still has to land somewhere
          VRHI_TRY(vrhi_buffer_create(g->dev, sizes[k], VRHI_STORAGE_BUFFER, slots[k]));
          g->temps.push_back(*slots[k]);
        }
      s.args.push_back(out_arg(oW, full));
      s.args.push_back(out_arg(ox, full));
      s.args.push_back(out_arg(ob, g->cols * 4));
      if (oL) s.args.push_back(out_arg(oL, 4));
      s.text = "mse_tanh_bwd stage 1 (hand-fused loss gradient: dW, dx, db" + std::string(oL ? ", loss)" : ")");
    } else {
      VRHI_TRY(vrhi_op_lookup("mse_tanh_fwd", &s.op));
      s.args.push_back(out_arg(oL, 4));
      s.text = "mse_tanh_fwd stage 1 (hand-fused loss)";
    }
    g->steps.push_back(s);
    *done = true;
    return VRHI_OK;
  }

  int emit_reduce(int i) {
    const Node &n = g->nodes[i];
    const int st = stage[i];
    const int in_shape = g->nodes[n.a].shape;
    auto rows_step = [&](const char *name, uint64_t r, uint64_t c, vrhi_arg in, vrhi_arg out, const char *what) -> int {
      Step s;
      s.stage = st;
      s.order = next_order++;
      VRHI_TRY(vrhi_op_lookup(name, &s.op));
      vrhi_rows_params rp{};
      rp.size = sizeof rp; rp.rows = r; rp.cols = c;
      s.params.assign((unsigned char *)&rp, (unsigned char *)&rp + sizeof rp);
      s.args = {in, out};
      std::ostringstream t;
      t << name << " stage " << st << " [" << r << "x" << c << "] " << what;
      s.text = t.str();
      g->steps.push_back(s);
      return VRHI_OK;
    };
    if (n.kind == K_SOFTMAX) return rows_step("row_softmax", g->rows, g->cols, arg_of(n.a, VRHI_INPUT), arg_of(i, VRHI_OUTPUT), "");
    switch (n.op) {
      case VRHI_R_ROW_SUM: return rows_step("row_sum", g->rows, g->cols, arg_of(n.a, VRHI_INPUT), arg_of(i, VRHI_OUTPUT), "");
      case VRHI_R_ROW_MAX: return rows_step("row_max", g->rows, g->cols, arg_of(n.a, VRHI_INPUT), arg_of(i, VRHI_OUTPUT), "");
      case VRHI_R_COL_SUM: return rows_step("col_sum", g->rows, g->cols, arg_of(n.a, VRHI_INPUT), arg_of(i, VRHI_OUTPUT), "");
      case VRHI_R_SUM_ALL:
      case VRHI_R_MEAN_ALL: {
        vrhi_arg flat_in = arg_of(n.a, VRHI_INPUT);
        uint64_t len = g->elems(in_shape);
        vrhi_arg dst = arg_of(i, VRHI_OUTPUT);
        auto mid_it = folded_mid.find(i);
        if (mid_it != folded_mid.end()) {  // the map kernel already left the column sums here
          vrhi_arg mid{}; mid.buffer = mid_it->second; mid.bytes = g->cols * 4; mid.arg_class = VRHI_INPUT;
          flat_in = mid;
          len = g->cols;
        } else if (in_shape == VRHI_SHAPE_FULL) {
          vrhi_buffer t = nullptr;
          VRHI_TRY(vrhi_buffer_create(g->dev, g->cols * 4, VRHI_STORAGE_BUFFER, &t));
          g->temps.push_back(t);
          vrhi_arg mid{}; mid.buffer = t; mid.bytes = g->cols * 4; mid.arg_class = VRHI_OUTPUT;
          VRHI_TRY(rows_step("col_sum", g->rows, g->cols, flat_in, mid, "(first half of a full sum)"));
          mid.arg_class = VRHI_INPUT;
          flat_in = mid;
          len = g->cols;
        }
        if (n.op == VRHI_R_SUM_ALL) return rows_step("row_sum", 1, len, flat_in, dst, "(flat sum)");
        // mean: flat sum into a temp, then scale by 1/N with a one-element map
        vrhi_buffer t2 = nullptr;
        VRHI_TRY(vrhi_buffer_create(g->dev, 16, VRHI_STORAGE_BUFFER, &t2));
        g->temps.push_back(t2);
        vrhi_arg sum{}; sum.buffer = t2; sum.bytes = 4; sum.arg_class = VRHI_OUTPUT;
        VRHI_TRY(rows_step("row_sum", 1, len, flat_in, sum, "(flat sum)"));
        Step s;
        s.stage = st;
        s.order = next_order++;
        VRHI_TRY(vrhi_op_lookup("map_tape", &s.op));
        vrhi_tape_params P{};
        P.size = sizeof P; P.n_inputs = 1; P.n_outputs = 1; P.n_instr = 2; P.rows = 1; P.cols = 1;
        P.instr[0].op = VRHI_T_CONST; P.instr[0].imm = (float)(1.0 / (double)g->elems(in_shape));
        P.instr[1].op = VRHI_T_MUL; P.instr[1].a = 0; P.instr[1].b = 1;
        P.out_value[0] = 2;
        s.params.assign((unsigned char *)&P, (unsigned char *)&P + sizeof P);
        sum.arg_class = VRHI_INPUT;
        s.args = {sum, dst};
        s.text = "map_tape    stage " + std::to_string(st) + " shape=scalar (mean = sum / N)";
        g->steps.push_back(s);
        return VRHI_OK;
      }
      default: return fail(VRHI_ERR_GRAPH, "unknown reduction %d", n.op);
    }
  }

  int run() {
    const int N = (int)g->nodes.size();
    for (auto b : g->temps) vrhi_buffer_destroy(b);
    g->temps.clear();
    g->steps.clear();
    g->plan.clear();
    if (g->outputs.empty()) return fail(VRHI_ERR_GRAPH, "the graph has no outputs");
    bool done = false;
    VRHI_TRY(try_mse(&done));
    if (!done) {
      live.assign(N, 0); root.assign(N, 0); stage.assign(N, -1); storage.assign(N, nullptr);
      for (auto &o : g->outputs) live[o.first] = 1;
      for (int i = N - 1; i >= 0; --i) {
        if (!live[i]) continue;
        const Node &n = g->nodes[i];
        if (n.a >= 0) live[n.a] = 1;
        if (n.b >= 0) live[n.b] = 1;
      }
      // roots: outputs and operands of reductions / softmax that are elementwise
      std::set<int> seen_out;
      for (auto &o : g->outputs) {
        const Node &n = g->nodes[o.first];
        if (n.kind == K_CONST) return fail(VRHI_ERR_GRAPH, "a constant cannot be a graph output");
        if (!seen_out.insert(o.first).second) return fail(VRHI_ERR_GRAPH, "node %d is bound to two output buffers", o.first);
        uint64_t sz = 0;
        vrhi_buffer_size(o.second, &sz);
        if (sz < g->elems(n.shape) * 4) return fail(VRHI_ERR_SIZE, "output buffer for node %d holds %llu bytes, %llu needed", o.first, (unsigned long long)sz, (unsigned long long)g->elems(n.shape) * 4);
        if (n.kind == K_INPUT) return fail(VRHI_ERR_GRAPH, "an input cannot be bound as an output");
        storage[o.first] = o.second;
        if (is_elementwise(n.kind)) root[o.first] = 1;
      }
      for (int i = 0; i < N; ++i) {
        if (!live[i]) continue;
        const Node &n = g->nodes[i];
        if (n.kind == K_INPUT) {
          if (!n.buf) return fail(VRHI_ERR_GRAPH, "input node %d has no buffer", i);
          storage[i] = n.buf;
        }
        if (n.kind == K_REDUCE || n.kind == K_SOFTMAX) {
          if (n.shape < 0) return fail(VRHI_ERR_GRAPH, "reduction %d cannot be applied to a %s operand", n.op, shape_name(g->nodes[n.a].shape));
          int a = n.a;
          if (g->nodes[a].kind == K_CONST) return fail(VRHI_ERR_GRAPH, "reduction of a constant");
          if (is_elementwise(g->nodes[a].kind)) root[a] = 1;
          if (!storage[i]) VRHI_TRY(temp_for(i));
        }
      }
      // A full-size elementwise value whose only reader is a column sum is never written: the map kernel
      // that computes it adds it up column by column (compiled tapes only, columns a multiple of 4).
      folded.clear(); folded_nodes.clear(); folded_mid.clear();
      if (g->cols % 4 == 0 && tape_jit_available()) {
        // readers that need the value in memory: reductions and softmax (elementwise readers recompute it
        // inside their own kernel from the leaves)
        std::vector<int> readers(N, 0);
        for (int i = 0; i < N; ++i) {
          if (!live[i]) continue;
          const Node &n = g->nodes[i];
          if (n.kind != K_REDUCE && n.kind != K_SOFTMAX) continue;
          if (n.a >= 0) ++readers[n.a];
        }
        for (int i = 0; i < N; ++i) {
          const Node &n = g->nodes[i];
          if (!live[i] || n.kind != K_REDUCE) continue;
          if (n.op != VRHI_R_COL_SUM && n.op != VRHI_R_SUM_ALL && n.op != VRHI_R_MEAN_ALL) continue;
          const int a = n.a;
          if (!is_elementwise(g->nodes[a].kind) || g->nodes[a].shape != VRHI_SHAPE_FULL) continue;
          if (readers[a] != 1 || seen_out.count(a) || storage[a] || folded.count(a)) continue;
          if (n.op == VRHI_R_COL_SUM) {
            folded[a] = storage[i];
            folded_nodes.insert(i);
          } else {  // a full sum is a column sum followed by a flat sum: the first half goes into the kernel
            vrhi_buffer t = nullptr;
            VRHI_TRY(vrhi_buffer_create(g->dev, g->cols * 4, VRHI_STORAGE_BUFFER, &t));
            g->temps.push_back(t);
            folded[a] = t;
            folded_mid[i] = t;
          }
        }
      }
      for (int i = 0; i < N; ++i)
        if (live[i] && root[i] && !storage[i] && !folded.count(i)) VRHI_TRY(temp_for(i));
      for (int i = 0; i < N; ++i)
        if (live[i]) node_stage(i);
      // group roots by (shape, stage), merging those that share a leaf or interior node
      std::vector<int> roots;
      for (int i = 0; i < N; ++i)
        if (live[i] && root[i]) roots.push_back(i);
      std::vector<char> used(roots.size(), 0);
      for (size_t k = 0; k < roots.size(); ++k) {
        if (used[k]) continue;
        used[k] = 1;
        std::vector<int> group{roots[k]};
        std::set<int> leaves, interior;
        collect(roots[k], leaves, interior);
        const int st = std::max(1, stage[roots[k]]);
        bool grew = true;
        while (grew) {
          grew = false;
          for (size_t m = k + 1; m < roots.size(); ++m) {
            if (used[m] || group.size() >= VRHI_TAPE_MAX_OUTPUTS) continue;
            const int r = roots[m];
            if (g->nodes[r].shape != g->nodes[roots[k]].shape || std::max(1, stage[r]) != st) continue;
            std::set<int> l2, i2;
            collect(r, l2, i2);
            bool share = false;
            for (int v : l2) if (leaves.count(v)) { share = true; break; }
            if (!share) for (int v : i2) if (interior.count(v)) { share = true; break; }
            if (!share) continue;
            std::set<int> lu = leaves, iu = interior;
            lu.insert(l2.begin(), l2.end());
            iu.insert(i2.begin(), i2.end());
            if (lu.size() > VRHI_TAPE_MAX_INPUTS || iu.size() > VRHI_TAPE_MAX_INSTR - 8) continue;
            leaves.swap(lu); interior.swap(iu);
            group.push_back(r);
            used[m] = 1;
            grew = true;
          }
        }
        VRHI_TRY(emit_map(group, leaves, st));
      }
      for (int i = 0; i < N; ++i)
        if (live[i] && (g->nodes[i].kind == K_REDUCE || g->nodes[i].kind == K_SOFTMAX)) {
          if (!folded_nodes.count(i)) VRHI_TRY(emit_reduce(i));
        }
      std::stable_sort(g->steps.begin(), g->steps.end(), [](const Step &x, const Step &y) {
        return x.stage != y.stage ? x.stage < y.stage : x.order < y.order;
      });
    }
    std::ostringstream plan;
    for (auto &s : g->steps) plan << s.text << "\n";
    g->plan = plan.str();
    g->compiled = true;
    return VRHI_OK;
  }
};

}  // namespace

extern "C" {

int vrhi_graph_create(vrhi_device dev, uint64_t rows, uint64_t cols, vrhi_graph *out_graph) {
  if (!dev || !out_graph) return fail(VRHI_ERR_INVALID, "NULL argument");
  *out_graph = nullptr;
  if (rows == 0 || cols == 0) return fail(VRHI_ERR_SIZE, "graph over an empty [%llu][%llu] shape", (unsigned long long)rows, (unsigned long long)cols);
  vrhi_graph_t *g = new (std::nothrow) vrhi_graph_t();
  if (!g) return fail(VRHI_ERR_OOM, "host allocation failed");
  g->dev = dev; g->rows = rows; g->cols = cols;
  static const bool no_specialize = [] { const char *e = getenv("VRHI_GRAPH_NO_SPECIALIZE"); return e && *e && *e != '0'; }();  // read once per process
  if (no_specialize) g->flags |= 1u;
  *out_graph = g;
  return VRHI_OK;
}

int vrhi_graph_destroy(vrhi_graph g) {
  if (!g) return VRHI_OK;
  for (auto b : g->temps) vrhi_buffer_destroy(b);
  delete g;
  return VRHI_OK;
}

int vrhi_graph_set_flags(vrhi_graph g, uint32_t flags) {
  if (!g) return fail(VRHI_ERR_INVALID, "NULL graph");
  g->flags = flags;
  g->compiled = false;
  return VRHI_OK;
}

int vrhi_graph_input(vrhi_graph g, vrhi_buffer buf, int shape, int *out_node) {
  if (!g || !buf || !out_node) return fail(VRHI_ERR_INVALID, "NULL argument");
  if (shape < VRHI_SHAPE_FULL || shape > VRHI_SHAPE_SCALAR) return fail(VRHI_ERR_INVALID, "shape %d out of range", shape);
  if (buf->dev != g->dev) return fail(VRHI_ERR_INVALID, "buffer lives on another device");
  if (buf->bytes < g->elems(shape) * 4) return fail(VRHI_ERR_SIZE, "input buffer holds %llu bytes, a %s input needs %llu", (unsigned long long)buf->bytes, shape_name(shape), (unsigned long long)g->elems(shape) * 4);
  Node n; n.kind = K_INPUT; n.shape = shape; n.buf = buf;
  *out_node = g->add(n);
  return VRHI_OK;
}

int vrhi_graph_const(vrhi_graph g, float value, int *out_node) {
  if (!g || !out_node) return fail(VRHI_ERR_INVALID, "NULL argument");
  *out_node = mk_const(g, value);
  return VRHI_OK;
}

static int arity_of(int op) {
  switch (op) {
    case VRHI_T_ADD: case VRHI_T_SUB: case VRHI_T_MUL: case VRHI_T_DIV: case VRHI_T_MAX: case VRHI_T_MIN: case VRHI_T_EQ: return 2;
    case VRHI_T_CONST: return 0;
    case VRHI_T_FMA: return 3;
    default: return (op > VRHI_T_FMA && op < VRHI_T_OPCOUNT) ? 1 : -1;
  }
}

int vrhi_graph_unary(vrhi_graph g, int tape_op, int a, int *out_node) {
  if (!g || !out_node) return fail(VRHI_ERR_INVALID, "NULL argument");
  if (arity_of(tape_op) != 1) return fail(VRHI_ERR_GRAPH, "op %d is not a unary elementwise op", tape_op);
  if (!g->valid(a)) return fail(VRHI_ERR_GRAPH, "operand %d is not a node of this graph", a);
  *out_node = mk_unary(g, tape_op, a);
  return VRHI_OK;
}

int vrhi_graph_binary(vrhi_graph g, int tape_op, int a, int b, int *out_node) {
  if (!g || !out_node) return fail(VRHI_ERR_INVALID, "NULL argument");
  if (arity_of(tape_op) != 2) return fail(VRHI_ERR_GRAPH, "op %d is not a binary elementwise op", tape_op);
  if (!g->valid(a) || !g->valid(b)) return fail(VRHI_ERR_GRAPH, "operand is not a node of this graph");
  *out_node = mk_binary(g, tape_op, a, b);
  return VRHI_OK;
}

int vrhi_graph_reduce(vrhi_graph g, int reduce_op, int a, int *out_node) {
  if (!g || !out_node) return fail(VRHI_ERR_INVALID, "NULL argument");
  if (!g->valid(a)) return fail(VRHI_ERR_GRAPH, "operand %d is not a node of this graph", a);
  if (reduce_op < VRHI_R_ROW_SUM || reduce_op > VRHI_R_MEAN_ALL) return fail(VRHI_ERR_GRAPH, "reduction %d out of range", reduce_op);
  if (reduce_shape(reduce_op, g->nodes[a].shape) < 0) return fail(VRHI_ERR_GRAPH, "reduction %d cannot be applied to a %s operand", reduce_op, shape_name(g->nodes[a].shape));
  *out_node = mk_reduce(g, reduce_op, a);
  return VRHI_OK;
}

int vrhi_graph_softmax(vrhi_graph g, int a, int *out_node) {
  if (!g || !out_node) return fail(VRHI_ERR_INVALID, "NULL argument");
  if (!g->valid(a)) return fail(VRHI_ERR_GRAPH, "operand %d is not a node of this graph", a);
  if (g->nodes[a].shape != VRHI_SHAPE_FULL) return fail(VRHI_ERR_GRAPH, "softmax needs a full [rows][cols] operand");
  Node n; n.kind = K_SOFTMAX; n.a = a; n.shape = VRHI_SHAPE_FULL;
  *out_node = g->add(n);
  return VRHI_OK;
}

int vrhi_graph_grad(vrhi_graph g, int loss_node, const int *wrt, int n_wrt, int *out_nodes) {
  if (!g || !wrt || !out_nodes || n_wrt <= 0) return fail(VRHI_ERR_INVALID, "bad argument");
  if (!g->valid(loss_node)) return fail(VRHI_ERR_GRAPH, "loss %d is not a node of this graph", loss_node);
  if (g->nodes[loss_node].shape != VRHI_SHAPE_SCALAR) return fail(VRHI_ERR_GRAPH, "the loss must be a scalar node (it is %s)", shape_name(g->nodes[loss_node].shape));
  for (int k = 0; k < n_wrt; ++k)
    if (!g->valid(wrt[k])) return fail(VRHI_ERR_GRAPH, "wrt[%d] = %d is not a node of this graph", k, wrt[k]);
  Autodiff ad{g, {}};
  return ad.run(loss_node, wrt, n_wrt, out_nodes);
}

int vrhi_graph_output(vrhi_graph g, int node, vrhi_buffer buf) {
  if (!g || !buf) return fail(VRHI_ERR_INVALID, "NULL argument");
  if (!g->valid(node)) return fail(VRHI_ERR_GRAPH, "node %d is not a node of this graph", node);
  if (buf->dev != g->dev) return fail(VRHI_ERR_INVALID, "buffer lives on another device");
  if (buf->cls == VRHI_INPUT || buf->cls == VRHI_UNIFORM || buf->cls == VRHI_UNIFORM_CONSTANT) return fail(VRHI_ERR_INVALID, "output buffer is read-only (class %s)", vrhi_arg_class_name(buf->cls));
  g->outputs.push_back({node, buf});
  g->compiled = false;
  return VRHI_OK;
}

int vrhi_graph_compile(vrhi_graph g) {
  if (!g) return fail(VRHI_ERR_INVALID, "NULL graph");
  Planner p;
  p.g = g;
  int rc = p.run();
  if (rc != VRHI_OK) g->compiled = false;
  return rc;
}

int vrhi_graph_launch(vrhi_graph g, vrhi_stream stream) {
  if (!g || !stream) return fail(VRHI_ERR_INVALID, "NULL argument");
  if (!g->compiled) return fail(VRHI_ERR_GRAPH, "the graph has not been compiled since it last changed");
  if (stream->dev != g->dev) return fail(VRHI_ERR_INVALID, "stream belongs to another device");
  for (auto &s : g->steps)
    VRHI_TRY(vrhi_op_launch(stream, s.op, s.args.data(), (int)s.args.size(), s.params.data(), s.params.size()));
  return VRHI_OK;
}

int vrhi_graph_describe(vrhi_graph g, char *out_text, size_t capacity, size_t *out_needed) {
  if (!g) return fail(VRHI_ERR_INVALID, "NULL graph");
  if (!g->compiled) return fail(VRHI_ERR_GRAPH, "the graph has not been compiled");
  if (out_needed) *out_needed = g->plan.size() + 1;
  if (out_text && capacity) {
    size_t n = std::min(capacity - 1, g->plan.size());
    memcpy(out_text, g->plan.data(), n);
    out_text[n] = 0;
  }
  return VRHI_OK;
}

int vrhi_graph_kernel_count(vrhi_graph g, int *out_count) {
  if (!g || !out_count) return fail(VRHI_ERR_INVALID, "NULL argument");
  if (!g->compiled) return fail(VRHI_ERR_GRAPH, "the graph has not been compiled");
  *out_count = (int)g->steps.size();
  return VRHI_OK;
}

}  // extern "C"
