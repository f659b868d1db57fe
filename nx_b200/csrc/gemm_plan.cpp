// Lowering of Nx `dot` nodes (nx/lib/nx.ex:13123-13161; EXLA: exla/lib/exla/defn.ex:1175-1197)
// to strided-batched matrix products.
#include <algorithm>

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
    Node wb;
    wb.op = "as_type";
    wb.dt = NXB_BF16;
    wb.shape = mul.shape;
    wb.args = {g.nodes[cvt].args[0]};
    g.nodes.push_back(wb);
    g.nodes[n].args[1] = (int)g.nodes.size() - 1;
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
