// Graph rewrites that run at compile time, before the lowering pass.
//
// GoMLX has fused ops for softmax, LayerNorm, GELU, Dense and attention, but RMSNorm reaches a backend as
// primitives: x * Rsqrt(ReduceSum(x * x, last) / C + eps) [* gamma], with the row statistic reshaped and broadcast
// back over the last axis somewhere along the way.  Run op by op that is three passes over x plus two over the
// output; the reference leaves the re-fusion to MPSGraph's closed compiler (mpsgraph function.go:2276-2565 only
// names the ops GoMLX already fuses).  RewriteRmsNorm recognises the pattern and turns its root into the single
// RmsNorm node the row kernel runs: one read of x, one write.
//
// The match is structural and conservative: anything it does not prove equal to RMSNorm over the LAST axis is left
// alone.  Statistics are then computed in fp32 with one final rounding, which for 16-bit inputs is more accurate
// than the op-by-op chain (each of whose results is rounded to 16 bits).
#include <cmath>
#include <cstring>
#include <unordered_map>
#include <unordered_set>

#include "common.h"

namespace b200 {

namespace {

float half_bits_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400u));
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

// The value of a one-element Constant seen through Cast / Reshape / BroadcastInDim / Identity.
bool ScalarValue(const Node* n, double* v) {
  while (n->op == Op::Cast || n->op == Op::Reshape || n->op == Op::BroadcastInDim || n->op == Op::Identity) n = n->in[0];
  if (n->op != Op::Constant || n->num_elements() != 1 || n->data.size() < (size_t)dtype_size(n->dtype)) return false;
  const uint8_t* p = n->data.data();
  switch (n->dtype) {
    case B200_FLOAT32: { float f; memcpy(&f, p, 4); *v = f; return true; }
    case B200_FLOAT64: { double d; memcpy(&d, p, 8); *v = d; return true; }
    case B200_BFLOAT16: { uint16_t h; memcpy(&h, p, 2); uint32_t b = (uint32_t)h << 16; float f; memcpy(&f, &b, 4); *v = f; return true; }
    case B200_FLOAT16: { uint16_t h; memcpy(&h, p, 2); *v = half_bits_to_float(h); return true; }
    case B200_INT32: { int32_t i; memcpy(&i, p, 4); *v = i; return true; }
    case B200_INT64: { int64_t i; memcpy(&i, p, 8); *v = (double)i; return true; }
    default: return false;
  }
}

std::vector<int64_t> NonUnit(const std::vector<int64_t>& d, size_t count) {
  std::vector<int64_t> r;
  for (size_t i = 0; i < count; ++i)
    if (d[i] != 1) r.push_back(d[i]);
  return r;
}

// A node holds one value per ROW of x (x viewed as [rows, C], C the last dim) if it is shaped like x without its last
// axis, up to size-1 dims ("stat"), or like x itself with every row constant ("full": a stat broadcast over the last axis).
struct RowShapes {
  const Node* x;
  std::vector<int64_t> stat;  // non-unit dims of x.dims[:-1]
  bool IsStat(const Node* n) const { return NonUnit(n->dims, n->dims.size()) == stat && n->num_elements() * x->dims.back() == x->num_elements(); }
  bool IsFull(const Node* n) const { return n->dims == x->dims; }
};

// value(n) = a * sum_j x[row, j]^2 + b for every row (or a * sum_j x[row, j] + b when matched with squared = false)
struct Affine {
  Node* x = nullptr;
  double a = 1, b = 0;
};

// Checks that a BroadcastInDim from a stat-shaped operand to x's shape keeps every row in place and only repeats along the last axis.
bool BroadcastKeepsRows(const Node* b, const Node* x) {
  const Node* src = b->in[0];
  const int r = x->rank();
  if (b->dims != x->dims || (int)b->ia.size() != src->rank()) return false;
  std::vector<int> want;  // x axes (last excluded) of non-unit size, in order
  for (int j = 0; j + 1 < r; ++j)
    if (x->dims[j] != 1) want.push_back(j);
  size_t k = 0;
  for (int i = 0; i < src->rank(); ++i) {
    if (src->dims[i] == 1) continue;
    if (k >= want.size() || b->ia[i] != want[k]) return false;
    ++k;
  }
  return k == want.size();
}

// A Reshape / Identity / BroadcastInDim between per-row values keeps every row's value in its row.
bool LayoutStepOk(const Node* l, const RowShapes& rs) {
  const Node* src = l->in[0];
  if (l->op != Op::BroadcastInDim) return rs.IsStat(l) || rs.IsFull(l);
  if (rs.IsFull(l)) return rs.IsFull(src) || (rs.IsStat(src) && BroadcastKeepsRows(l, rs.x));
  if (rs.IsStat(l) && rs.IsStat(src)) {  // only adds unit dims; the non-unit dims must keep their order
    int64_t last = -1;
    for (int i = 0; i < src->rank(); ++i) {
      if (src->dims[i] == 1) continue;
      if (l->ia[i] <= last) return false;
      last = l->ia[i];
    }
    return true;
  }
  return false;
}

// Proves value(n) = a * rowsumsq(x) + b.  On the way down x is unknown, so shapes are validated on the way back up.
bool MatchAffine(Node* n, Affine* out, RowShapes* rs, int depth = 0, bool squared = true) {
  if (depth > 16) return false;
  auto shaped = [&](Node* m) { return rs->IsStat(m) || rs->IsFull(m); };
  switch (n->op) {
    case Op::Reshape:
    case Op::Identity:
    case Op::BroadcastInDim:
      return MatchAffine(n->in[0], out, rs, depth + 1, squared) && LayoutStepOk(n, *rs);
    case Op::Reduce: {
      Node* sq = n->in[0];
      if (n->ia.size() != 2 || n->ia[0] != B200_REDUCE_SUM || sq->rank() < 1 || n->ia[1] != sq->rank() - 1) return false;
      if (squared && (sq->op != Op::Mul || sq->in[0] != sq->in[1])) return false;
      Node* x = squared ? sq->in[0] : sq;
      if (x->dims.back() < 2) return false;
      out->x = x; out->a = 1; out->b = 0;
      rs->x = x;
      rs->stat = NonUnit(x->dims, x->dims.size() - 1);
      return true;
    }
    case Op::Add:
    case Op::Sub:
    case Op::Mul:
    case Op::Div: {
      double c;
      Node* u = nullptr;
      bool const_first = false;
      if (ScalarValue(n->in[1], &c)) u = n->in[0];
      else if (ScalarValue(n->in[0], &c)) { u = n->in[1]; const_first = true; }
      else return false;
      if (const_first && (n->op == Op::Sub || n->op == Op::Div)) return false;
      if (!MatchAffine(u, out, rs, depth + 1, squared) || !shaped(n)) return false;
      switch (n->op) {
        case Op::Add: out->b += c; break;
        case Op::Sub: out->b -= c; break;
        case Op::Mul: out->a *= c; out->b *= c; break;
        default:
          if (c == 0) return false;
          out->a /= c; out->b /= c;
      }
      return true;
    }
    default:
      return false;
  }
}

// q = rsqrt(affine) per row, seen through layout ops: Rsqrt(u), or 1 / Sqrt(u).
bool MatchInvRoot(Node* q, Affine* aff, RowShapes* rs) {
  std::vector<Node*> layout;
  while (q->op == Op::Reshape || q->op == Op::BroadcastInDim || q->op == Op::Identity) { layout.push_back(q); q = q->in[0]; }
  Node* inner = nullptr;
  double one;
  if (q->op == Op::Rsqrt) inner = q->in[0];
  else if (q->op == Op::Div && ScalarValue(q->in[0], &one) && one == 1.0 && q->in[1]->op == Op::Sqrt) inner = q->in[1]->in[0];
  if (!inner || !MatchAffine(inner, aff, rs)) return false;
  if (!(rs->IsStat(q) || rs->IsFull(q))) return false;
  for (Node* l : layout)
    if (!LayoutStepOk(l, *rs)) return false;
  return true;
}

// n_hat = x * q (either order) or x / Sqrt(affine).  Fills x and epsilon.
bool MatchNormalized(Node* m, Node** x, double* eps) {
  if (!dtype_is_float(m->dtype) || m->dtype == B200_FLOAT64) return false;
  Affine aff;
  RowShapes rs{};
  bool ok = false;
  if (m->op == Op::Mul) {
    for (int side = 0; side < 2 && !ok; ++side) {
      aff = Affine();
      ok = MatchInvRoot(m->in[1 - side], &aff, &rs) && aff.x == m->in[side];
    }
  } else if (m->op == Op::Div) {
    Node* q = m->in[1];
    std::vector<Node*> layout;
    while (q->op == Op::Reshape || q->op == Op::BroadcastInDim || q->op == Op::Identity) { layout.push_back(q); q = q->in[0]; }
    if (q->op == Op::Sqrt && MatchAffine(q->in[0], &aff, &rs) && aff.x == m->in[0] && (rs.IsStat(q) || rs.IsFull(q))) {
      ok = true;
      for (Node* l : layout) ok = ok && LayoutStepOk(l, rs);
    }
  }
  if (!ok || m->dims != aff.x->dims || m->dtype != aff.x->dtype) return false;
  const double C = (double)aff.x->dims.back();
  // mean of squares: a = 1 / C up to the rounding of a float32 (or 16-bit) constant
  if (!(aff.a > 0) || std::fabs(aff.a * C - 1.0) > 4e-3) return false;
  if (!(aff.b >= 0) || !std::isfinite(aff.b)) return false;
  *x = aff.x;
  *eps = aff.b;
  return true;
}

// G = gamma[C] broadcast over the rows of x: BroadcastInDim(g, {last}) (seen through reshapes that only add unit dims).
Node* MatchGamma(Node* G, const Node* x) {
  if (G->dims != x->dims) return nullptr;
  if (G->op != Op::BroadcastInDim) return nullptr;
  Node* g = G->in[0];
  const int r = x->rank();
  // every non-unit operand dim must land on the last axis
  int non_unit = 0;
  for (int i = 0; i < g->rank(); ++i) {
    if (g->dims[i] == 1) continue;
    if (G->ia[i] != r - 1) return nullptr;
    ++non_unit;
  }
  if (non_unit != 1 || g->num_elements() != x->dims.back()) return nullptr;
  while ((g->op == Op::Reshape || g->op == Op::Identity) && g->in[0]->num_elements() == g->num_elements()) g = g->in[0];
  if (g->dtype != x->dtype) return nullptr;
  return g;
}

}  // namespace

namespace {
// nodes reachable from the targets, and their users among those
void LiveAndUsers(Graph& graph, const std::vector<Node*>& targets, std::unordered_set<Node*>* live,
                  std::unordered_map<Node*, std::vector<Node*>>* users) {
  std::vector<Node*> stack(targets.begin(), targets.end());
  while (!stack.empty()) {
    Node* n = stack.back();
    stack.pop_back();
    if (!live->insert(n).second) continue;
    for (Node* i : n->in) stack.push_back(i);
  }
  for (auto& up : graph.nodes)
    if (live->count(up.get()))
      for (Node* i : up->in) (*users)[i].push_back(up.get());
}
}  // namespace

// A transformer block ends its attention and MLP halves with "x + Dense(...)" (and a gated MLP multiplies two Dense
// results: the same rewrite with * in place of +).  Run op by op the sum costs a read of
// both operands and a write of the result (three passes over the activations) right after the GEMM wrote one of them;
// in the GEMM's epilogue it costs one extra read.  The product is still rounded to the storage type before the
// addition, so the fused value is bit-identical to the two-op one.
int RewriteGemmResidual(Graph& graph, const std::vector<Node*>& targets) {
  std::unordered_set<Node*> live;
  std::unordered_map<Node*, std::vector<Node*>> users;
  LiveAndUsers(graph, targets, &live, &users);
  std::unordered_set<Node*> is_target(targets.begin(), targets.end());
  int rewritten = 0;
  for (auto& up : graph.nodes) {
    Node* m = up.get();
    if (!live.count(m) || (m->op != Op::Add && m->op != Op::Mul)) continue;
    if (!(m->dtype == B200_FLOAT32 || m->dtype == B200_BFLOAT16 || m->dtype == B200_FLOAT16)) continue;
    for (int side = 0; side < 2; ++side) {
      Node* x = m->in[side];
      Node* r = m->in[1 - side];
      if (x == r || r->dims != m->dims || r->dtype != m->dtype) continue;
      {
        // a broadcast or generated operand is cheaper inside an elementwise kernel (stride 0, no tensor in memory)
        const Node* rs = r;
        while (rs->op == Op::Reshape || rs->op == Op::Identity || rs->op == Op::Cast) rs = rs->in[0];
        if (rs->op == Op::BroadcastInDim || rs->op == Op::Constant || rs->op == Op::Iota) continue;
      }
      // the product, seen through views that keep the element order, each with this chain as its only user
      bool chain_ok = true;
      Node* d = x;
      while (d->op == Op::Reshape || d->op == Op::Identity) {
        if (is_target.count(d) || users[d].size() != 1) { chain_ok = false; break; }
        d = d->in[0];
      }
      if (!chain_ok || d->op != Op::DotGeneral || is_target.count(d) || users[d].size() != 1) continue;
      if (d->dtype != m->dtype || d->num_elements() != m->num_elements()) continue;
      if (d->fa.size() > 1 && d->fa[1] != 0) continue;   // already carries a residual
      // r must exist independently of d (it cannot use d: d has a single user, the chain)
      m->in = d->in;
      m->in.push_back(r);
      m->ia = d->ia;
      m->fa = {d->fa.empty() ? 0.0 : d->fa[0], m->op == Op::Mul ? 2.0 : 1.0};   // before m->op changes below
      m->op = Op::DotGeneral;
      ++rewritten;
      break;
    }
  }
  return rewritten;
}

// Rotary position embedding in its rotate-half form reaches a backend as
//   Add(Mul(x, cos), Mul(Concatenate(Slice(x, upper half), Slice(x, lower half)), sin))        (last axis, even size)
// with the sign of the rotation folded into the sin table (or into a Neg that this matcher does not look through).
// Op by op that is two slice copies, a concatenation and a three-op elementwise pass over every query and key of
// every layer; as one Rope node the kernel reads x once (in place inside the QKV projection when it can) and writes
// the result once.  Each product and the sum are rounded to the storage type, so the value is the op-by-op one.
int RewriteRope(Graph& graph, const std::vector<Node*>& targets) {
  std::unordered_set<Node*> live;
  std::unordered_map<Node*, std::vector<Node*>> users;
  LiveAndUsers(graph, targets, &live, &users);
  auto half_slice = [](Node* s, Node* x, bool upper) {
    if (s->op != Op::Slice || s->in[0] != x) return false;
    const int r = x->rank();
    const int64_t D = x->dims[r - 1], h = D / 2;
    for (int d = 0; d < r; ++d) {
      const int64_t start = s->ia[2 * d], stride = s->ia[2 * d + 1];
      if (stride != 1) return false;
      if (d < r - 1) {
        if (start != 0 || s->dims[d] != x->dims[d]) return false;
      } else if (start != (upper ? h : 0) || s->dims[d] != h) {
        return false;
      }
    }
    return true;
  };
  int rewritten = 0;
  for (auto& up : graph.nodes) {
    Node* m = up.get();
    if (!live.count(m) || m->op != Op::Add) continue;
    if (!(m->dtype == B200_FLOAT32 || m->dtype == B200_BFLOAT16 || m->dtype == B200_FLOAT16)) continue;
    const int r = m->rank();
    if (r < 1 || m->dims[r - 1] % 16 != 0) continue;   // half a head is a whole number of 16-byte vectors for every float type
    Node* p = m->in[0];
    Node* q = m->in[1];
    if (p->op != Op::Mul || q->op != Op::Mul) continue;
    Node *x = nullptr, *c = nullptr, *s = nullptr;
    // one product has the Concatenate of x's halves as an operand, the other has x itself
    for (int which = 0; which < 2 && !x; ++which) {
      Node* rot_mul = which ? p : q;
      Node* dir_mul = which ? q : p;
      for (int rs = 0; rs < 2 && !x; ++rs) {
        Node* w = rot_mul->in[rs];
        if (w->op != Op::Concatenate || w->in.size() != 2 || w->ia.empty() || w->ia[0] != r - 1) continue;
        Node* src = w->in[0]->op == Op::Slice ? w->in[0]->in[0] : nullptr;
        if (!src || src->dims != m->dims || src->dtype != m->dtype) continue;
        if (!half_slice(w->in[0], src, true) || !half_slice(w->in[1], src, false)) continue;
        for (int ds = 0; ds < 2; ++ds) {
          if (dir_mul->in[ds] != src) continue;
          x = src;
          c = dir_mul->in[1 - ds];
          s = rot_mul->in[1 - rs];
          break;
        }
      }
    }
    if (!x || c->dims != m->dims || s->dims != m->dims || c->dtype != m->dtype || s->dtype != m->dtype) continue;
    m->op = Op::Rope;
    m->in = {x, c, s};
    m->ia.clear();
    m->fa.clear();
    ++rewritten;
  }
  return rewritten;
}

int RewriteRmsNorm(Graph& graph, const std::vector<Node*>& targets) {
  // nodes reachable from the targets, and their users
  std::unordered_set<Node*> live;
  std::vector<Node*> stack(targets.begin(), targets.end());
  while (!stack.empty()) {
    Node* n = stack.back();
    stack.pop_back();
    if (!live.insert(n).second) continue;
    for (Node* i : n->in) stack.push_back(i);
  }
  std::unordered_map<Node*, std::vector<Node*>> users;
  for (auto& up : graph.nodes)
    if (live.count(up.get()))
      for (Node* i : up->in) users[i].push_back(up.get());
  std::unordered_set<Node*> is_target(targets.begin(), targets.end());

  int rewritten = 0;
  for (auto& up : graph.nodes) {
    Node* m = up.get();
    if (!live.count(m) || (m->op != Op::Mul && m->op != Op::Div)) continue;
    Node* x = nullptr;
    double eps = 0;
    if (!MatchNormalized(m, &x, &eps)) continue;
    Node* root = m;
    Node* gamma = nullptr;
    auto& mu = users[m];
    if (!is_target.count(m) && mu.size() == 1 && mu[0]->op == Op::Mul && mu[0]->dtype == m->dtype) {
      Node* u = mu[0];
      Node* G = u->in[0] == m ? u->in[1] : u->in[0];
      if (G != m) {
        if (Node* g = MatchGamma(G, x)) {
          // gamma must exist before the node that will read it; it does, being an operand of u (created after its operands)
          root = u;
          gamma = g;
        }
      }
    }
    // LayerNorm spelled in primitives is the same pattern one level up: the normalised value is d = x0 - mean(x0), i.e.
    // Sub(x0, M) with M = rowsum(x0) / C per row (ref mpsgraph function.go:2430-2558 is this very chain, two-pass).
    Node* x0 = nullptr;
    if (x->op == Op::Sub && x->in[0]->dims == x->dims && x->in[0]->dtype == x->dtype) {
      Affine mean;
      RowShapes mrs{};
      const double C = (double)x->dims.back();
      if (MatchAffine(x->in[1], &mean, &mrs, 0, /*squared=*/false) && mean.x == x->in[0] && (mrs.IsStat(x->in[1]) || mrs.IsFull(x->in[1])) &&
          std::fabs(mean.a * C - 1.0) <= 4e-3 && mean.b == 0.0)
        x0 = x->in[0];
    }
    Node* beta = nullptr;
    if (x0 && !is_target.count(root)) {
      // ... [* gamma] + beta: an Add of a vector broadcast over the rows
      auto& ru = users[root];
      if (ru.size() == 1 && ru[0]->op == Op::Add && ru[0]->dtype == root->dtype) {
        Node* u = ru[0];
        Node* B = u->in[0] == root ? u->in[1] : u->in[0];
        if (B != root) {
          if (Node* b = MatchGamma(B, x)) {
            root = u;
            beta = b;
          }
        }
      }
    }
    root->op = x0 ? Op::LayerNorm : Op::RmsNorm;
    root->in = {x0 ? x0 : x};
    if (gamma) root->in.push_back(gamma);
    if (beta) root->in.push_back(beta);
    root->ia = {gamma ? 1 : 0, beta ? 1 : 0, (int64_t)x->rank() - 1};
    root->fa = {eps};
    ++rewritten;
  }
  return rewritten;
}

// Softmax spelled in primitives (what a model emits when a backend does not list FusedSoftmax):
//   e = Exp(Sub(x, M)),  M = ReduceMax(x, last) kept / broadcast per row;   y = Div(e, S),  S = ReduceSum(e, last) per row.
// Op by op that is two reductions and three elementwise passes; as one Softmax node the row kernel reads x once and
// writes y once.  The row kernel computes the same max-subtracted form in fp32 with one final rounding.
int RewriteSoftmax(Graph& graph, const std::vector<Node*>& targets) {
  std::unordered_set<Node*> live;
  std::unordered_map<Node*, std::vector<Node*>> users;
  LiveAndUsers(graph, targets, &live, &users);
  // n = Reduce(type, last axis)(src) seen through layout ops that keep every row's value in its row
  auto row_reduce = [](Node* n, int type, const Node* like) -> Node* {
    std::vector<Node*> layout;
    while (n->op == Op::Reshape || n->op == Op::BroadcastInDim || n->op == Op::Identity) { layout.push_back(n); n = n->in[0]; }
    if (n->op != Op::Reduce || n->ia.size() != 2 || n->ia[0] != type) return nullptr;
    Node* src = n->in[0];
    if (src->rank() < 1 || n->ia[1] != src->rank() - 1 || src->dims != like->dims) return nullptr;
    RowShapes rs{src, NonUnit(src->dims, src->dims.size() - 1)};
    if (!rs.IsStat(n)) return nullptr;
    for (Node* l : layout)
      if (!LayoutStepOk(l, rs)) return nullptr;
    return src;
  };
  int rewritten = 0;
  for (auto& up : graph.nodes) {
    Node* m = up.get();
    if (!live.count(m) || m->op != Op::Div) continue;
    if (!(m->dtype == B200_FLOAT32 || m->dtype == B200_BFLOAT16 || m->dtype == B200_FLOAT16)) continue;
    Node* e = m->in[0];
    if (e->op != Op::Exp || e->dims != m->dims || e->dtype != m->dtype || m->rank() < 1 || m->dims.back() < 2) continue;
    if (row_reduce(m->in[1], B200_REDUCE_SUM, e) != e) continue;
    Node* d = e->in[0];
    if (d->op != Op::Sub || d->in[0]->dims != m->dims || d->in[0]->dtype != m->dtype) continue;
    Node* x = d->in[0];
    if (row_reduce(d->in[1], B200_REDUCE_MAX, x) != x) continue;
    m->op = Op::Softmax;
    m->in = {x};
    m->ia = {(int64_t)m->rank() - 1};
    m->fa.clear();
    ++rewritten;
  }
  return rewritten;
}

}  // namespace b200
