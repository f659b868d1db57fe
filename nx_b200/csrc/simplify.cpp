// Algebraic rewrites of a parsed graph, applied before planning.
//
// share_shifted_exp_sums: Nx.logsumexp (nx/lib/nx.ex:18400-18433) shifts by
//     m0 = select(is_infinity(m), 0, m),   m = reduce_max(x, axes, keep_axes: true)
// and sums exp(x - m0).  A softmax over the same axes of the same tensor sums exp(x - m).  Where m
// is finite the two sums are the same number, computed twice: a second exponential per element.
// Where m is infinite the first sum is known without looking at the elements: m = +inf means some
// element is +inf and none is NaN (the maximum propagates NaN, and NaN is not infinite), so
// sum(exp(x - 0)) = +inf; m = -inf means every element is -inf, so the sum is 0.  Hence
//     sum(exp(x - m0)) = select(is_infinity(m), select(m > 0, +inf, 0), sum(exp(x - m)))
// exactly (the finite case is the same accumulation as the softmax's), and the second exponential
// disappears from the generated kernel.
#include <limits>
#include <map>

#include "program.h"

namespace nxb {
namespace {

int skip_meta(const Graph& g, int n) {
  while (g.nodes[n].op == "metadata") n = g.nodes[n].args[0];
  return n;
}

bool is_zero_constant(const Node& c) {
  if (c.op != "constant") return false;
  if (!c.flts.empty()) return c.flts[0] == 0.0;
  return !c.ints.empty() && c.ints[0] == 0;
}

struct Match {
  int r1 = -1;       // sum(exp(x - m))
  int mask = -1;     // is_infinity(m)
  int rm = -1;       // m
};

}  // namespace

void share_shifted_exp_sums(Graph& g) {
  const size_t N = g.nodes.size();
  std::vector<int> uses(N, 0);
  for (size_t n = 0; n < N; ++n) for (int a : g.nodes[n].args) uses[a]++;
  for (int o : g.outputs) uses[o]++;

  std::map<int, Match> found;
  for (size_t r = 0; r < N; ++r) {
    const Node& R = g.nodes[r];
    if (R.op != "sum" || !dtype_is_float(R.dt) || R.args.size() != 1 || R.ints.size() < 2) continue;
    const int e2 = R.args[0];
    const Node& E2 = g.nodes[e2];
    if (E2.op != "exp" || uses[e2] != 1 || E2.dt != R.dt) continue;
    const Node& S2 = g.nodes[E2.args[0]];
    if (S2.op != "subtract" || uses[E2.args[0]] != 1 || S2.dt != R.dt) continue;
    const int x = S2.args[0];
    if (g.nodes[x].shape != S2.shape || g.nodes[x].dt != R.dt) continue;
    const int m0 = skip_meta(g, S2.args[1]);
    const Node& M0 = g.nodes[m0];
    if (M0.op != "select" || M0.args.size() != 3 || M0.dt != R.dt) continue;
    const int mask = M0.args[0];
    if (g.nodes[mask].op != "is_infinity" || !is_zero_constant(g.nodes[skip_meta(g, M0.args[1])])) continue;
    const int rm = skip_meta(g, M0.args[2]);
    const Node& RM = g.nodes[rm];
    if (RM.op != "reduce_max" || RM.args[0] != x || RM.ints.size() != R.ints.size() || RM.ints[0] != 1 || RM.dt != R.dt) continue;
    if (skip_meta(g, g.nodes[mask].args[0]) != rm || g.nodes[mask].shape != RM.shape || M0.shape != RM.shape) continue;
    bool same_axes = true;
    for (size_t i = 1; i < R.ints.size(); ++i) same_axes = same_axes && R.ints[i] == RM.ints[i];
    if (!same_axes) continue;
    // the softmax's sum: an earlier node sum(exp(x - m)) over the same axes
    for (size_t c = 0; c < r; ++c) {
      const Node& R1 = g.nodes[c];
      if (R1.op != "sum" || R1.dt != R.dt || R1.ints.size() != R.ints.size()) continue;
      bool ax = true;
      for (size_t i = 1; i < R.ints.size(); ++i) ax = ax && R1.ints[i] == R.ints[i];
      if (!ax) continue;
      const Node& E1 = g.nodes[R1.args[0]];
      if (E1.op != "exp" || E1.dt != R.dt) continue;
      const Node& S1 = g.nodes[E1.args[0]];
      if (S1.op != "subtract" || S1.dt != R.dt || S1.args[0] != x || skip_meta(g, S1.args[1]) != rm) continue;
      Match mt;
      mt.r1 = (int)c;
      mt.mask = mask;
      mt.rm = rm;
      found[(int)r] = mt;
      break;
    }
  }
  if (found.empty()) return;

  // rebuild the node list: the helper nodes of a rewritten sum go directly before it, so that every
  // node still follows its arguments
  std::vector<Node> out;
  out.reserve(N + 8 * found.size());
  std::vector<int> remap(N, -1);
  auto push = [&](Node nd) { out.push_back(std::move(nd)); return (int)out.size() - 1; };
  for (size_t n = 0; n < N; ++n) {
    auto it = found.find((int)n);
    if (it == found.end()) {
      Node nd = g.nodes[n];
      for (int& a : nd.args) a = remap[a];
      remap[n] = push(std::move(nd));
      continue;
    }
    const Node& R = g.nodes[n];
    const Match& mt = it->second;
    auto shaped = [&](int old_node) {          // the node's value with the shape of R (kept axes dropped or not)
      const Node& src = g.nodes[old_node];
      if (src.shape == R.shape) return remap[old_node];
      Node rs;
      rs.op = "reshape";
      rs.dt = src.dt;
      rs.shape = R.shape;
      rs.args = {remap[old_node]};
      return push(std::move(rs));
    };
    auto scalar = [&](double v) {
      Node c;
      c.op = "constant";
      c.dt = R.dt;
      c.flts = {v};
      return push(std::move(c));
    };
    const int mask_r = shaped(mt.mask), m_r = shaped(mt.rm), sum_r = shaped(mt.r1);
    const int zero = scalar(0.0), inf = scalar(std::numeric_limits<double>::infinity());
    Node gt;
    gt.op = "greater";
    gt.dt = NXB_U8;
    gt.shape = R.shape;
    gt.args = {m_r, zero};
    const int gt_i = push(std::move(gt));
    Node inner;
    inner.op = "select";
    inner.dt = R.dt;
    inner.shape = R.shape;
    inner.args = {gt_i, inf, zero};
    const int inner_i = push(std::move(inner));
    Node sel;
    sel.op = "select";
    sel.dt = R.dt;
    sel.shape = R.shape;
    sel.args = {mask_r, inner_i, sum_r};
    remap[n] = push(std::move(sel));
  }
  for (int& o : g.outputs) o = remap[o];
  g.nodes = std::move(out);
}

}  // namespace nxb
