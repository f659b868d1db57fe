// Lowering of Nx `dot` nodes (nx/lib/nx.ex:13123-13161; EXLA: exla/lib/exla/defn.ex:1175-1197)
// to strided-batched matrix products.
#include <algorithm>
#include <cstdlib>
#include <set>

#include "gemm.h"

namespace nxb {

namespace {
struct DotAxes { std::vector<int> c1, b1, c2, b2; };

DotAxes dot_axes(const Node& nd) {
  DotAxes d;
  size_t p = 0;
  std::vector<int>* lists[4] = {&d.c1, &d.b1, &d.c2, &d.b2};
  for (auto* l : lists) {
    int64_t n = nd.ints.at(p++);
    for (int64_t i = 0; i < n; ++i) l->push_back((int)nd.ints.at(p++));
  }
  return d;
}

// Can `shape`, with the given batch / contract axes, be read as [batch][free][contract]
// (returns 1) or [batch][contract][free] (returns 2) without moving data?  0 otherwise.
int classify(const std::vector<int64_t>& shape, const std::vector<int>& batch, const std::vector<int>& contract,
             const std::vector<int>& want_contract_order) {
  int r = (int)shape.size(), nb = (int)batch.size(), nc = (int)contract.size();
  for (int i = 0; i < nb; ++i) if (batch[i] != i) return 0;
  // contract axes must be adjacent, ascending, and in the pairing order
  for (int i = 0; i + 1 < nc; ++i) if (contract[i + 1] != contract[i] + 1) return 0;
  (void)want_contract_order;
  if (nc == 0) return 1;
  if (contract[0] + nc == r) return 1;       // trailing
  if (contract[0] == nb) return 2;           // right after the batch axes
  return 0;
}
}  // namespace

// Rewrites the operands of every dot so that each is [batch][free][contract] or
// [batch][contract][free]; inserts a transpose node where the data has to move.
void canonicalize_dots(Graph& g) {
  size_t N = g.nodes.size();
  for (size_t n = 0; n < N; ++n) {
    if (g.nodes[n].op != "dot") continue;
    DotAxes d = dot_axes(g.nodes[n]);
    for (int side = 0; side < 2; ++side) {
      std::vector<int>& con = side ? d.c2 : d.c1;
      std::vector<int>& bat = side ? d.b2 : d.b1;
      int arg = g.nodes[n].args[side];
      std::vector<int64_t> shape = g.nodes[arg].shape;
      if (classify(shape, bat, con, con)) continue;
      // transpose to [batch][free][contract]
      std::vector<int> perm = bat;
      for (int j = 0; j < (int)shape.size(); ++j)
        if (!std::count(bat.begin(), bat.end(), j) && !std::count(con.begin(), con.end(), j)) perm.push_back(j);
      for (int c : con) perm.push_back(c);
      Node t;
      t.op = "transpose";
      t.dt = g.nodes[arg].dt;
      for (int p : perm) { t.shape.push_back(shape[p]); t.ints.push_back(p); }
      t.args = {arg};
      g.nodes.push_back(t);
      int tn = (int)g.nodes.size() - 1;
      g.nodes[n].args[side] = tn;
      int r = (int)shape.size(), nc = (int)con.size(), nb = (int)bat.size();
      for (int i = 0; i < nb; ++i) bat[i] = i;
      for (int i = 0; i < nc; ++i) con[i] = r - nc + i;
    }
    std::vector<int64_t> ints;
    for (auto* l : {&d.c1, &d.b1, &d.c2, &d.b2}) {
      ints.push_back((int64_t)l->size());
      for (int v : *l) ints.push_back(v);
    }
    g.nodes[n].ints = ints;
  }
}

// Weight-only quantised linear: dot(x: bf16, multiply(as_type(W: s8 -> f32), S)) where S has
// one value per output channel.  The per-channel factor does not depend on the contracted
// index, so it moves out of the sum:  sum_k x[m,k] * (W[n,k] * S[n]) = S[n] * sum_k x[m,k] * W[n,k].
// The product then runs on the tensor cores with W converted (exactly) to bf16, f32
// accumulation, and S applied to the accumulator in the epilogue.
void rewrite_quantised_linears(Graph& g) {
  size_t N = g.nodes.size();
  auto skip_meta = [&](int n) { while (g.nodes[n].op == "metadata") n = g.nodes[n].args[0]; return n; };
  for (size_t n = 0; n < N; ++n) {
    if (g.nodes[n].op != "dot" || g.nodes[n].dt != NXB_F32) continue;
    DotAxes d = dot_axes(g.nodes[n]);
    if (!d.b1.empty() || d.c1.size() != 1 || d.c2.size() != 1) continue;
    int x = g.nodes[n].args[0], wq = skip_meta(g.nodes[n].args[1]);
    if (g.nodes[x].dt != NXB_BF16 || g.nodes[x].shape.size() != 2) continue;
    const Node& mul = g.nodes[wq];
    if (mul.op != "multiply" || mul.dt != NXB_F32 || mul.shape.size() != 2) continue;
    int cvt = -1, sc = -1;
    for (int side = 0; side < 2; ++side) {
      int f = skip_meta(mul.args[side]);
      if (g.nodes[f].op == "as_type" && g.nodes[g.nodes[f].args[0]].dt == NXB_S8 && g.nodes[f].shape == mul.shape) { cvt = f; sc = skip_meta(mul.args[1 - side]); }
    }
    if (cvt < 0) continue;
    const int caxis = d.c2[0], faxis = 1 - caxis;
    const Node& S = g.nodes[sc];
    if (S.dt != NXB_F32) continue;
    // S aligned to the right of {d0,d1}: extent 1 (or absent) along the contracted axis, N along the free one
    std::vector<int64_t> sh = S.shape;
    while (sh.size() < 2) sh.insert(sh.begin(), 1);
    if (sh.size() != 2 || sh[caxis] != 1 || sh[faxis] != mul.shape[faxis]) continue;
    if (mul.shape[caxis] % 8 != 0) continue;      // the tensor-core path needs 16-byte aligned rows
    // Few rows of x and W stored {N,K}: the product kernel converts W itself, so the layer reads
    // the s8 weights once and no 16-bit copy of them is ever written.
    const bool in_kernel = !getenv("NXB200_NO_INLINE_DEQUANT") && caxis == 1 && d.c1[0] == 1 && g.nodes[x].shape[0] >= 1 &&
                           g.nodes[x].shape[0] <= WQ_LINEAR_MAX_ROWS && mul.shape[caxis] % 16 == 0;
    if (in_kernel) {
      g.nodes[n].args[1] = g.nodes[cvt].args[0];
    } else {
      Node wb;
      wb.op = "as_type";
      wb.dt = NXB_BF16;
      wb.shape = mul.shape;
      wb.args = {g.nodes[cvt].args[0]};
      g.nodes.push_back(wb);
      g.nodes[n].args[1] = (int)g.nodes.size() - 1;
    }
    g.nodes[n].args.push_back(sc);      // third argument: keeps the factor alive and ordered before the product
    g.nodes[n].scale_arg = sc;
  }
  // dot(as_type(a: s8 -> s32), as_type(b: s8 -> s32)) -> the s8 tensor-core product with an s32
  // accumulator: the same integers, bit for bit (|sum| <= k * 127^2 stays far inside 32 bits for
  // any k the tensor map can address... guarded below).
  for (size_t n = 0; n < N; ++n) {
    Node& nd = g.nodes[n];
    if (nd.op != "dot" || nd.dt != NXB_S32 || nd.scale_arg >= 0) continue;
    int a = skip_meta(nd.args[0]), b = skip_meta(nd.args[1]);
    auto widened_s8 = [&](int x) {
      return g.nodes[x].op == "as_type" && g.nodes[x].dt == NXB_S32 && g.nodes[g.nodes[x].args[0]].dt == NXB_S8;
    };
    if (!widened_s8(a) || !widened_s8(b)) continue;
    DotAxes d = dot_axes(nd);
    int64_t k = 1;
    for (int ax : d.c1) k *= g.nodes[a].shape[ax];
    if (k % 16 != 0 || k > 130000) continue;       // 16-byte rows; 130000 * 127^2 < 2^31
    nd.args[0] = g.nodes[a].args[0];
    nd.args[1] = g.nodes[b].args[0];
  }
}

// Attention:  dot(q,k) -> X = elementwise(scores, indices ...) -> softmax over the key axis ->
// dot(p,v), with every intermediate private to the chain, becomes ONE node that the fused
// kernel of attn_sm100_device.cuh executes (the scores never reach memory).  `X`'s subgraph is
// kept and compiled into the kernel as the score transform.
// attention node: args = {q, k, v, extra buffers of the transform...};
//                 ints = {X node, scores dot node, causal, Sq, Sk}.
void rewrite_attention(Graph& g) {
  if (getenv("NXB200_NO_FUSED_ATTENTION")) return;
  const size_t N = g.nodes.size();
  std::vector<int> uses(N, 0);
  for (size_t n = 0; n < N; ++n) for (int a : g.nodes[n].args) uses[a]++;
  for (int o : g.outputs) uses[o]++;
  auto is_last_axis_keep = [&](const Node& nd, size_t rank) {
    return nd.ints.size() == 3 && nd.ints[0] == 1 && nd.ints[1] == 1 && nd.ints[2] == (int64_t)rank - 1;
  };
  for (size_t n = 0; n < N; ++n) {
    if (g.nodes[n].op != "dot" || g.nodes[n].dt != NXB_BF16) continue;
    const Node& D2 = g.nodes[n];
    DotAxes d2 = dot_axes(D2);
    const int p = D2.args[0], v = D2.args[1];
    const Node& P = g.nodes[p];
    const size_t r = P.shape.size();
    if (r < 2 || g.nodes[v].shape.size() != r || P.op != "divide" || uses[p] != 1) continue;
    std::vector<int> lead;
    for (size_t i = 0; i + 2 < r; ++i) lead.push_back((int)i);
    if (d2.c1 != std::vector<int>{(int)r - 1} || d2.c2 != std::vector<int>{(int)r - 2} || d2.b1 != lead || d2.b2 != lead) continue;
    const int e = P.args[0], sm = P.args[1];
    const Node& S = g.nodes[sm];
    const Node& E = g.nodes[e];
    if (S.op != "sum" || !is_last_axis_keep(S, r) || S.args[0] != e || uses[sm] != 1) continue;
    if (E.op != "exp" || uses[e] != 2) continue;
    const Node& SUB = g.nodes[E.args[0]];
    if (SUB.op != "subtract" || uses[E.args[0]] != 1) continue;
    const int x = SUB.args[0], mx = SUB.args[1];
    const Node& M = g.nodes[mx];
    if (M.op != "reduce_max" || !is_last_axis_keep(M, r) || M.args[0] != x || uses[mx] != 1 || uses[x] != 2) continue;
    const Node& X = g.nodes[x];
    if (X.shape != P.shape || X.dt != NXB_BF16 || E.dt != NXB_BF16 || P.dt != NXB_BF16) continue;
    // the transform's subgraph: exactly one product, no reductions, private intermediates
    std::vector<int> stack{x}, cone_nodes, extras;
    std::set<int> seen;
    int d1 = -1;
    bool ok = true;
    std::map<int, int> refs;
    while (!stack.empty() && ok) {
      int c = stack.back();
      stack.pop_back();
      if (!seen.insert(c).second) continue;
      const Node& cn = g.nodes[c];
      if (cn.op == "dot") { if (d1 >= 0 && d1 != c) ok = false; d1 = c; continue; }
      if (cn.op == "parameter" || cn.op == "tensor" || cn.op == "concatenate" || cn.op == "all_reduce" || cn.op == "attention") { extras.push_back(c); continue; }
      if (cn.op == "sum" || cn.op == "product" || cn.op == "reduce_max" || cn.op == "reduce_min" || cn.op == "all" || cn.op == "any" ||
          cn.op == "argmax" || cn.op == "argmin") { ok = false; break; }
      cone_nodes.push_back(c);
      for (int a : cn.args) { refs[a]++; stack.push_back(a); }
    }
    if (!ok || d1 < 0 || uses[d1] != refs[d1] || extras.size() > 10) continue;
    const Node& D1 = g.nodes[d1];
    DotAxes a1 = dot_axes(D1);
    const int q = D1.args[0], k = D1.args[1];
    if (g.nodes[q].shape.size() != r || g.nodes[k].shape.size() != r || D1.shape != X.shape || D1.dt != NXB_BF16) continue;
    if (a1.c1 != std::vector<int>{(int)r - 1} || a1.c2 != std::vector<int>{(int)r - 1} || a1.b1 != lead || a1.b2 != lead) continue;
    if (g.nodes[q].dt != NXB_BF16 || g.nodes[k].dt != NXB_BF16 || g.nodes[v].dt != NXB_BF16) continue;
    const int64_t D = g.nodes[q].shape[r - 1], Sq = g.nodes[q].shape[r - 2], Sk = g.nodes[k].shape[r - 2];
    if (D != 128 || g.nodes[v].shape[r - 1] != 128 || g.nodes[v].shape[r - 2] != Sk) continue;
    int64_t bh = 1;
    for (size_t i = 0; i + 2 < r; ++i) bh *= g.nodes[q].shape[i];
    if (bh < 1 || bh > 65535 * 8 || Sq < 1 || Sk < 1) continue;
    // causal: X = select(broadcast(iota(rows) >= iota(cols)), ., -inf)
    int causal = 0;
    if (X.op == "select" && Sq == Sk) {
      int mk = X.args[0];
      while (g.nodes[mk].op == "broadcast" || g.nodes[mk].op == "metadata") {
        const Node& b = g.nodes[mk];
        if (b.op == "broadcast") {
          // must map the mask's two axes onto the last two axes of the scores
          if (b.ints.size() != 3 || b.ints[1] != (int64_t)r - 2 || b.ints[2] != (int64_t)r - 1) break;
        }
        mk = b.args[0];
      }
      const Node& ge = g.nodes[mk];
      const Node& neg = g.nodes[X.args[2]];
      const bool neg_inf = neg.op == "constant" && !neg.flts.empty() && neg.flts[0] < -1e300;
      if (ge.op == "greater_equal" && ge.shape == std::vector<int64_t>{Sq, Sk} && neg_inf) {
        const Node& i0 = g.nodes[ge.args[0]];
        const Node& i1 = g.nodes[ge.args[1]];
        if (i0.op == "iota" && i1.op == "iota" && i0.ints[0] == 0 && i1.ints[0] == 1 && i0.shape == ge.shape && i1.shape == ge.shape) causal = 1;
      }
    }
    Node A;
    A.op = "attention";
    A.dt = NXB_BF16;
    A.shape = D2.shape;
    A.args = {q, k, v};
    for (int ex : extras) A.args.push_back(ex);
    // {batch, head, rows, 128}: the head transposes around the attention are folded into its addressing.
    // v = transpose({batch, key, head, 128}, [0,2,1,3]) is read in place through a four-dimensional tensor
    // map; a result whose only reader is transpose(., [0,2,1,3]) is written in that order directly.
    const std::vector<int64_t> swap12{0, 2, 1, 3};
    int64_t heads = 1, v_bshd = 0;
    int vsrc = v;
    if (r == 4) {
      heads = D2.shape[1];
      const Node& V = g.nodes[v];
      if (V.op == "transpose" && V.ints == swap12 && g.nodes[V.args[0]].dt == NXB_BF16) { vsrc = V.args[0]; v_bshd = 1; }
    }
    A.args[2] = vsrc;
    A.ints = {x, d1, causal, Sq, Sk, heads, v_bshd, 0};
    g.nodes[n] = A;
    // the product that computed the scores is no longer part of the program
    for (int a : g.nodes[d1].args) uses[a]--;
    if (r == 4 && uses[n] == 1) {
      for (size_t t = n + 1; t < N; ++t) {
        Node& T = g.nodes[t];
        if (T.op != "transpose" || T.args.size() != 1 || T.args[0] != (int)n || T.ints != swap12) continue;
        Node B = g.nodes[n];
        B.shape = T.shape;
        B.ints[7] = 1;
        g.nodes[t] = B;                  // the transpose IS the attention now; node n is dead
        break;
      }
    }
  }
}

bool plan_dot(Plan& plan, int node, std::vector<int>& need, GemmSpec* out) {
  Graph& g = plan.g;
  const Node& nd = g.nodes[node];
  DotAxes d = dot_axes(nd);
  const Node& a = g.nodes[nd.args[0]];
  const Node& b = g.nodes[nd.args[1]];
  int ca = classify(a.shape, d.b1, d.c1, d.c1), cb = classify(b.shape, d.b2, d.c2, d.c2);
  if (!ca || !cb) fail(NXB_ERR_RUNTIME, "internal: dot operands were not canonicalised");
  GemmSpec gs;
  gs.batch = 1;
  for (int ax : d.b1) gs.batch *= a.shape[ax];
  gs.k = 1;
  for (int ax : d.c1) gs.k *= a.shape[ax];
  gs.m = shape_numel(a.shape) / std::max<int64_t>(1, gs.batch * gs.k);
  gs.n = shape_numel(b.shape) / std::max<int64_t>(1, gs.batch * gs.k);
  if (gs.batch == 0 || gs.k == 0) { gs.m = gs.batch ? shape_numel(a.shape) / gs.batch : 0; }
  gs.a.dt = a.dt;
  gs.b.dt = b.dt;
  gs.a.trans = ca == 2;
  gs.b.trans = cb == 2;          // [batch][contract][free] = [k][n]: n contiguous
  gs.a.ld = gs.a.trans ? gs.m : gs.k;
  gs.b.ld = gs.b.trans ? gs.n : gs.k;
  gs.a.batch_stride = gs.m * gs.k;
  gs.b.batch_stride = gs.n * gs.k;
  gs.a.slot = a.slot;
  gs.b.slot = b.slot;
  gs.out_slot = nd.slot;
  gs.out_dt = nd.dt;
  if (a.slot < 0) need.push_back(nd.args[0]);
  if (b.slot < 0) need.push_back(nd.args[1]);
  if (nd.scale_arg >= 0) {
    gs.scale_slot = g.nodes[nd.scale_arg].slot;
    if (gs.scale_slot < 0) need.push_back(nd.scale_arg);
  }
  gs.desc = "gemm#" + std::to_string(node) + " batch=" + std::to_string(gs.batch) + " m=" + std::to_string(gs.m) + " n=" +
            std::to_string(gs.n) + " k=" + std::to_string(gs.k) + " a=" + dtype_name(a.dt) + (gs.a.trans ? "[k,m]" : "[m,k]") + " b=" +
            dtype_name(b.dt) + (gs.b.trans ? "[k,n]" : "[n,k]") + " out=" + dtype_name(nd.dt) +
            (nd.scale_arg >= 0 ? " epilogue=per-column f32 scale" : "");
  *out = gs;
  return true;
}

}  // namespace nxb
