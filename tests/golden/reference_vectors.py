"""Known-answer vectors transcribed from the reference's own test files.

Each case names the file and lines it was read from.  ``fun`` builds the graph
with the nx_b200 front-end exactly as the reference test's ``defn`` does with
Nx; ``args`` are ``(nested_list, type)`` pairs; ``expect`` is one
``(nested_list, type)`` per output.  ``exact`` cases must match bit for bit
(NaN == NaN, as Nx.Testing.assert_equal does, nx/lib/nx/testing.ex:22-68);
the others use the reference's assert_all_close tolerance
(atol = rtol = 1e-4, nx/lib/nx/testing.ex:151-154).

The same list is used twice: to pin the CPU oracle (no GPU needed) and, in
the GPU tests, to check the CUDA path through the C ABI.
"""
from nx_b200 import nx

INF, NAN = float("inf"), float("nan")

CASES = []


def case(name, cite, fun, args, expect, exact=True, modes=("xla_like", "binary_backend")):
    CASES.append(dict(name=name, cite=cite, fun=fun, args=args, expect=expect, exact=exact, modes=modes))


T3 = [[[1, 2, 3], [4, 5, 6]], [[7, 8, 9], [10, 11, 12]]]

# ---- sum: exla/test/exla/defn/expr_test.exs:1978-2024 ---------------------------------
case("sum s32", "exla/test/exla/defn/expr_test.exs:1982", lambda t: nx.sum(t), [([1, 2, 3], "s32")], [(6, "s32")])
case("sum s8 -> s32", "exla/test/exla/defn/expr_test.exs:1983", lambda t: nx.sum(t), [([1, 2, 3], "s8")], [(6, "s32")])
case("sum u8 -> u32", "exla/test/exla/defn/expr_test.exs:1984", lambda t: nx.sum(t), [([1, 2, 3], "u8")], [(6, "u32")])
case("sum f32", "exla/test/exla/defn/expr_test.exs:1985-1990", lambda t: nx.sum(t), [([1.0, 2.0, 3.0], "f32")], [(6.0, "f32")])
case("sum axis 1", "exla/test/exla/defn/expr_test.exs:1997-2000", lambda t: nx.sum(t, axes=[1]), [(T3, "s32")],
     [([[5, 7, 9], [17, 19, 21]], "s32")])
case("sum axis -3", "exla/test/exla/defn/expr_test.exs:2001", lambda t: nx.sum(t, axes=[-3]), [(T3, "s32")],
     [([[8, 10, 12], [14, 16, 18]], "s32")])
case("sum axes 1,-3", "exla/test/exla/defn/expr_test.exs:2002", lambda t: nx.sum(t, axes=[1, -3]), [(T3, "s32")],
     [([22, 26, 30], "s32")])
case("sum of equal does not overflow", "exla/test/exla/defn/expr_test.exs:2005-2011",
     lambda t: nx.sum(nx.equal(t, 1.0)), [([1, 1, 1], "s32")], [(3, "u32")])
case("sum keep_axes", "exla/test/exla/defn/expr_test.exs:2017", lambda t: nx.sum(t, keep_axes=True),
     [([1, 2, 3], "s32")], [([6], "s32")])
case("sum axes 0,2 keep", "exla/test/exla/defn/expr_test.exs:2020-2023",
     lambda t: nx.sum(t, axes=[0, 2], keep_axes=True),
     [([[[1, 2, 3], [4, 5, 6]], [[1, 2, 3], [4, 5, 6]]], "s32")], [([[[12], [30]]], "s32")])

# ---- reduce_max: exla/test/exla/defn/expr_test.exs:2137-2184 ----------------------------
case("reduce_max s32", "exla/test/exla/defn/expr_test.exs:2141", lambda t: nx.reduce_max(t), [([1, 2, 3], "s32")], [(3, "s32")])
case("reduce_max s8", "exla/test/exla/defn/expr_test.exs:2143-2146", lambda t: nx.reduce_max(t), [([1, 2, 3], "s8")], [(3, "s8")])
case("reduce_max u8", "exla/test/exla/defn/expr_test.exs:2148-2151", lambda t: nx.reduce_max(t), [([1, 2, 3], "u8")], [(3, "u8")])
case("reduce_max f32", "exla/test/exla/defn/expr_test.exs:2153-2158", lambda t: nx.reduce_max(t), [([1.0, 2.0, 3.0], "f32")], [(3.0, "f32")])
case("reduce_max axis 1", "exla/test/exla/defn/expr_test.exs:2165-2168", lambda t: nx.reduce_max(t, axes=[1]), [(T3, "s32")],
     [([[4, 5, 6], [10, 11, 12]], "s32")])
case("reduce_max axes 1,-3", "exla/test/exla/defn/expr_test.exs:2170", lambda t: nx.reduce_max(t, axes=[1, -3]), [(T3, "s32")],
     [([10, 11, 12], "s32")])
case("reduce_max axes 0,2 keep", "exla/test/exla/defn/expr_test.exs:2180-2183",
     lambda t: nx.reduce_max(t, axes=[0, 2], keep_axes=True),
     [([[[1, 2, 3], [4, 5, 6]], [[1, 2, 3], [4, 5, 6]]], "s32")], [([[[3], [6]]], "s32")])

# ---- argmax / argmin: exla/test/exla/defn/expr_test.exs:2239-2307 -----------------------
for ty in ("s32", "s8", "u8", "f32", "bf16"):
    case(f"argmax {ty}", "exla/test/exla/defn/expr_test.exs:2250-2256", lambda t: nx.argmax(t), [([1, 2, 3], ty)], [(2, "s32")])
    case(f"argmin {ty}", "exla/test/exla/defn/expr_test.exs:2260-2266", lambda t: nx.argmin(t), [([1, 2, 3], ty)], [(0, "s32")])
case("argmax flat", "exla/test/exla/defn/expr_test.exs:2256", lambda t: nx.argmax(t), [([[1, 2, 3], [4, 5, 6]], "s32")], [(5, "s32")])
case("argmax axis 1", "exla/test/exla/defn/expr_test.exs:2269-2274", lambda t: nx.argmax(t, axis=1),
     [([[[1, 1, 1], [1, 1, 3]], [[6, 2, 3], [2, 8, 3]]], "s32")], [([[0, 0, 1], [0, 1, 0]], "s32")])
case("argmin axis 1", "exla/test/exla/defn/expr_test.exs:2276-2281", lambda t: nx.argmin(t, axis=1),
     [([[[4, 2, 3], [1, -5, 3]], [[6, 2, 3], [4, 8, 3]]], "s32")], [([[1, 1, 0], [1, 0, 0]], "s32")])
case("argmax tie low", "exla/test/exla/defn/expr_test.exs:2284", lambda t: nx.argmax(t, axis=1),
     [([[1, 2, 2], [1, 2, 2]], "s32")], [([1, 1], "s32")])
case("argmax tie high", "exla/test/exla/defn/expr_test.exs:2285", lambda t: nx.argmax(t, axis=1, tie_break="high"),
     [([[1, 2, 2], [1, 2, 2]], "s32")], [([2, 2], "s32")])
case("argmax keep_axis", "exla/test/exla/defn/expr_test.exs:2288-2296", lambda t: nx.argmax(t, axis=1, keep_axis=True),
     [([[[4, 2, 3], [1, -5, 3]], [[6, 2, 3], [4, 8, 3]]], "s32")], [([[[0, 0, 0]], [[0, 1, 0]]], "s32")])
case("argmin keep_axis", "exla/test/exla/defn/expr_test.exs:2298-2306", lambda t: nx.argmin(t, axis=1, keep_axis=True),
     [([[[4, 2, 3], [1, -5, 3]], [[6, 2, 3], [4, 8, 3]]], "s32")], [([[[1, 1, 0]], [[1, 0, 0]]], "s32")])

NONFINITE = [[-INF, INF, 1], [-INF, NAN, 1], [-INF, -INF, 1], [-INF, 0, 1], [INF, INF, 1], [INF, NAN, 1],
             [INF, -INF, 1], [INF, 0, 1], [NAN, INF, 1], [NAN, NAN, 1], [NAN, -INF, 1], [NAN, 0, 1]]
# The two-NaN row (index 9) is where BinaryBackend's scan order shows: it
# returns the last NaN.  EXLA's reducer is order dependent there, so the row is
# only pinned for the BinaryBackend mode (and the CUDA path follows it).
case("argmax non-finite", "nx/test/nx_test.exs:1778-1798", lambda t: nx.argmax(t, axis=1), [(NONFINITE, "f32")],
     [([1, 1, 2, 2, 0, 1, 0, 0, 0, 1, 0, 0], "s32")], modes=("binary_backend",))
case("argmin non-finite", "nx/test/nx_test.exs:1746-1766", lambda t: nx.argmin(t, axis=1), [(NONFINITE, "f32")],
     [([0, 1, 0, 0, 2, 1, 1, 1, 0, 1, 0, 0], "s32")], modes=("binary_backend",))

# ---- dot: exla/test/exla/defn/expr_test.exs:2603-2695 ------------------------------------
case("dot scalars", "exla/test/exla/defn/expr_test.exs:2607-2609", lambda a, b: nx.dot(a, b), [(-2.0, "f32"), (-2, "s32")], [(4.0, "f32")])
case("dot vectors s32", "exla/test/exla/defn/expr_test.exs:2613-2616", lambda a, b: nx.dot(a, b),
     [([1, 2, 3], "s32"), ([4, 5, 6], "s32")], [(32, "s32")])
case("dot vectors f32 x s32", "exla/test/exla/defn/expr_test.exs:2618-2621", lambda a, b: nx.dot(a, b),
     [([1.0, 2.0, 3.0], "f32"), ([4, 5, 6], "s32")], [(32.0, "f32")])
case("dot matrices s32", "exla/test/exla/defn/expr_test.exs:2627-2633", lambda a, b: nx.dot(a, b),
     [([[1, 2, 3], [4, 5, 6]], "s32"), ([[7, 8], [9, 10], [11, 12]], "s32")], [([[58, 64], [139, 154]], "s32")])
case("dot matrices f32", "exla/test/exla/defn/expr_test.exs:2635-2641", lambda a, b: nx.dot(a, b),
     [([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], "f32"), ([[7.0, 8.0], [9.0, 10.0], [11.0, 12.0]], "f32")],
     [([[58.0, 64.0], [139.0, 154.0]], "f32")])
case("dot matrices f32 x s32", "exla/test/exla/defn/expr_test.exs:2643-2649", lambda a, b: nx.dot(a, b),
     [([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], "f32"), ([[7, 8], [9, 10], [11, 12]], "s32")],
     [([[58.0, 64.0], [139.0, 154.0]], "f32")])
case("dot tensors", "exla/test/exla/defn/expr_test.exs:2652-2671", lambda a, b: nx.dot(a, b),
     [([[[1, 2, 3], [4, 5, 6], [7, 8, 9]], [[1, 2, 3], [4, 5, 6], [7, 8, 9]]], "s32"),
      ([[[1, 2, 3], [3, 4, 5], [5, 6, 7]]], "s32")],
     [([[[[22, 28, 34]], [[49, 64, 79]], [[76, 100, 124]]], [[[22, 28, 34]], [[49, 64, 79]], [[76, 100, 124]]]], "s32")])
case("batched dot", "exla/test/exla/defn/expr_test.exs:2673-2684",
     lambda a, b: nx.dot(a, [1], [0], b, [1], [0]),
     [([[[0, 1, 2], [3, 4, 5]], [[6, 7, 8], [9, 10, 11]], [[12, 13, 14], [15, 16, 17]]], "f32"),
      ([[[0, 1], [2, 3]], [[4, 5], [6, 7]], [[8, 9], [10, 11]]], "f32")],
     [([[[6.0, 9.0], [8.0, 13.0], [10.0, 17.0]], [[78.0, 93.0], [88.0, 105.0], [98.0, 117.0]],
        [[246.0, 273.0], [264.0, 293.0], [282.0, 313.0]]], "f32")])


def _iota_list(shape):
    import numpy as np
    return np.arange(int(np.prod(shape))).reshape(shape).tolist()


case("general dot", "exla/test/exla/defn/expr_test.exs:2686-2694",
     lambda a, b: nx.dot(a, [0, 1], [], b, [1, 2], []),
     [(_iota_list((4, 5, 2)), "f32"), (_iota_list((2, 4, 5)), "f32")], [([[4940.0, 12540.0], [5130.0, 13130.0]], "f32")])
case("dot/6 batched doc example", "nx/lib/nx.ex:13040-13054",
     lambda u, v: nx.dot(u, [2], [0], v, [1], [0]),
     [([[[1, 1]], [[2, 2]]], "s32"), ([[[3], [3]], [[4], [4]]], "s32")], [([[[6]], [[16]]], "s32")])
case("bf16 dot = 14", "exla/test/exla/defn/expr_test.exs:4275-4283", lambda a, b: nx.dot(a, b),
     [([1, 2, 3], "bf16"), ([1, 2, 3], "bf16")], [(14, "bf16")])

# ---- as_type, bf16, select: exla/test/exla/defn/expr_test.exs ---------------------------
case("as_type s32 -> f32", "exla/test/exla/defn/expr_test.exs:1111-1113", lambda t: nx.as_type(t, "f32"),
     [([1, 2, 3], "s32")], [([1.0, 2.0, 3.0], "f32")])
case("as_type non-finite -> u8", "exla/test/exla/defn/expr_test.exs:1121-1124", lambda t: nx.as_type(t, "u8"),
     [([INF, NAN, -INF], "f32")], [([255, 0, 0], "u8")])
case("as_type non-finite -> s16", "exla/test/exla/defn/expr_test.exs:1126-1129", lambda t: nx.as_type(t, "s16"),
     [([INF, NAN, -INF], "f32")], [([32767, 0, -32768], "s16")])
case("bf16 add", "exla/test/exla/defn/expr_test.exs:4247-4255", lambda a, b: a + b,
     [([1.0, 2.0, 3.0], "bf16"), ([4.0, 5.0, 6.0], "bf16")], [([5.0, 7.0, 9.0], "bf16")])
case("select scalar pred", "exla/test/exla/defn/expr_test.exs:765-769", lambda p, a, b: nx.select(p, a, b),
     [(1, "s32"), ([1, 2, 3], "s32"), ([4, 5, 6], "s32")], [([1, 2, 3], "s32")])
case("select merges types", "exla/test/exla/defn/expr_test.exs:781-788", lambda p, a, b: nx.select(p, a, b),
     [(1, "s32"), ([1, 2, 3], "u8"), ([4, 5, 6], "f32")], [([1.0, 2.0, 3.0], "f32")])
case("select broadcast", "exla/test/exla/defn/expr_test.exs:792-795", lambda p, a, b: nx.select(p, a, b),
     [([1, 0, 1, 0, 1], "s32"), ([10], "s32"), ([1, 2, 3, 4, 5], "s32")], [([10, 2, 10, 4, 10], "s32")])
case("select non-zero is true", "exla/test/exla/defn/expr_test.exs:797-800", lambda p, a, b: nx.select(p, a, b),
     [([-2, -1, 0, 1, 2], "s32"), ([10], "s32"), ([1, 2, 3, 4, 5], "s32")], [([10, 10, 3, 10, 10], "s32")])
case("add s32", "exla/test/exla/defn/expr_test.exs:175", lambda a, b: a + b, [([1, 2], "s32"), ([3, 4], "s32")], [([4, 6], "s32")])
case("add u8 + (-3) -> s16", "exla/test/exla/defn/expr_test.exs:179-208 (types per nx/lib/nx/type.ex:536-566)",
     lambda a: a + (-3), [([1, 2], "u8")], [([-2, -1], "s16")])
case("add u8 + 3.0 -> f32", "exla/test/exla/defn/expr_test.exs:179-208", lambda a: a + 3.0, [([1, 2], "u8")], [([4.0, 5.0], "f32")])
case("add f32 + u16", "exla/test/exla/defn/expr_test.exs:179-208", lambda a, b: a + b,
     [([1, 2], "f32"), (3, "u16")], [([4.0, 5.0], "f32")])

# ---- softmax, logsumexp ---------------------------------------------------------------------
case("softmax", "exla/test/exla/defn/expr_test.exs:3057-3071", lambda t: nx.exp(t) / nx.sum(nx.exp(t)),
     [([1.0, 2.0, 3.0, 4.0], "f32")],
     [([0.03205860328008499, 0.08714431874203257, 0.23688281808991013, 0.6439142598879722], "f32")], exact=False)
case("logsumexp removes axes", "nx/test/nx_test.exs:3516-3530", lambda t: nx.logsumexp(t, axes=[2]),
     [([[[11.0], [12.0], [13.0]]], "f32")], [([[11.0, 12.0, 13.0]], "f32")])
LSE_IN = [[INF, INF, INF], [INF, INF, -INF], [INF, INF, 0.0], [INF, -INF, INF], [INF, -INF, -INF], [INF, -INF, 0.0],
          [INF, 0.0, INF], [INF, 0.0, -INF], [INF, 0.0, 0.0], [-INF, INF, INF], [-INF, INF, -INF], [-INF, INF, 0.0],
          [-INF, -INF, INF], [-INF, -INF, -INF], [-INF, -INF, 0.0], [-INF, 0.0, INF], [-INF, 0.0, -INF],
          [-INF, 0.0, 0.0], [0.0, INF, INF], [0.0, INF, -INF], [0.0, INF, 0.0], [0.0, -INF, INF], [0.0, -INF, -INF],
          [0.0, -INF, 0.0], [0.0, 0.0, INF], [0.0, 0.0, -INF]]
LSE_OUT = [INF] * 13 + [-INF, 0.0, INF, 0.0, 0.6931471824645996, INF, INF, INF, INF, 0.0, 0.6931471824645996, INF,
                        0.6931471824645996]
case("logsumexp infinities", "nx/test/nx_test.exs:3532-3593", lambda t: nx.logsumexp(t, axes=[1]),
     [(LSE_IN, "f32")], [(LSE_OUT, "f32")])
case("logsumexp doc all", "nx/lib/nx.ex:18340-18344", lambda t: nx.logsumexp(t), [([[1, 2], [3, 4], [5, 6]], "s32")],
     [(6.4561934, "f32")], exact=False)
case("logsumexp doc axis y", "nx/lib/nx.ex:18353-18358", lambda t: nx.logsumexp(t, axes=[1]), [([[1, 2], [3, 4], [5, 6]], "s32")],
     [([2.3132617, 4.3132615, 6.3132615], "f32")], exact=False)
case("logsumexp doc axes x,z keep", "nx/lib/nx.ex:18368-18379", lambda t: nx.logsumexp(t, axes=[0, 2], keep_axes=True),
     [([[[1, 2], [3, 4]], [[5, 6], [7, 8]]], "s32")], [([[[6.3314114], [8.331411]]], "f32")], exact=False)
case("logsumexp scaling factor", "nx/lib/nx.ex:18333-18339",
     lambda t, a: nx.logsumexp(t, exp_scaling_factor=a),
     [([1, 2, 3, 4, 5, 6], "s32"), ([-1, -1, -1, 1, 1, 1], "s32")], [(6.356537, "f32")], exact=False)

# ---- gather / take: exla/test/exla/defn/expr_test.exs:3398-3496, nx/lib/nx.ex:14554-14640,15036-15111 ----
T2 = [[1, 2], [3, 4]]
T222 = [[[1, 2], [11, 12]], [[101, 102], [111, 112]]]
case("gather 1d result", "exla/test/exla/defn/expr_test.exs:3464-3467", lambda t, i: nx.gather(t, i),
     [(T2, "s32"), ([[1, 1], [0, 1], [1, 0]], "s32")], [([4, 2, 3], "s32")])
case("gather rank 3", "exla/test/exla/defn/expr_test.exs:3469-3475", lambda t, i: nx.gather(t, i),
     [(T222, "s32"), ([[0, 0, 0], [0, 1, 1], [1, 1, 1]], "s32")], [([1, 12, 112], "s32")])
case("gather clamps out-of-range indices", "exla/test/exla/defn/expr_test.exs:3477-3480", lambda t, i: nx.gather(t, i),
     [(T2, "s32"), ([[-1, -1], [10, 11], [-1, 10]], "s32")], [([1, 4, 2], "s32")], modes=("xla_like",))
case("gather 2d result", "exla/test/exla/defn/expr_test.exs:3483-3488", lambda t, i: nx.gather(t, i),
     [(T2, "s32"), ([[[1, 1], [0, 0]], [[1, 0], [0, 1]]], "s32")], [([[4, 1], [3, 2]], "s32")])
case("gather subsets", "nx/lib/nx.ex:15061-15069", lambda t, i: nx.gather(t, i),
     [([[1, 2, 3], [3, 4, 5]], "s32"), ([[1], [0]], "s32")], [([[3, 4, 5], [1, 2, 3]], "s32")])
case("gather axes: [1]", "nx/lib/nx.ex:15075-15085", lambda t, i: nx.gather(t, i, axes=[1]),
     [([[1, 2, 3], [4, 5, 6]], "s32"), ([[1], [0], [2], [1]], "s32")], [([[2, 5], [1, 4], [3, 6], [2, 5]], "s32")])
case("gather axes: [2] of iota {2,1,3}", "nx/lib/nx.ex:15091-15111", lambda t, i: nx.gather(t, i, axes=[2]),
     [([[[0, 1, 2]], [[3, 4, 5]]], "s32"), ([[[1], [0], [2]]], "s32")], [([[[[1], [4]], [[0], [3]], [[2], [5]]]], "s32")])
case("take axis 0", "exla/test/exla/defn/expr_test.exs:3403-3406", lambda t, i: nx.take(t, i),
     [(T2, "s32"), ([1, 0, 1], "s32")], [([[3, 4], [1, 2], [3, 4]], "s32")])
case("take axis 1", "exla/test/exla/defn/expr_test.exs:3408-3411", lambda t, i: nx.take(t, i, axis=1),
     [(T2, "s32"), ([1, 0, 1], "s32")], [([[2, 1, 2], [4, 3, 4]], "s32")])
case("take rank 3 axis 1", "nx/lib/nx.ex:14585-14601", lambda t, i: nx.take(t, i, axis=1),
     [(T222, "s32"), ([1, 0, 1], "s32")], [([[[11, 12], [1, 2], [11, 12]], [[111, 112], [101, 102], [111, 112]]], "s32")])
case("take 2d indices", "exla/test/exla/defn/expr_test.exs:3414-3456", lambda t, i: nx.take(t, i, axis=1),
     [(T222, "s32"), ([[0, 0, 0], [1, 1, 1], [0, 0, 0]], "s32")],
     [([[[[1, 2]] * 3, [[11, 12]] * 3, [[1, 2]] * 3], [[[101, 102]] * 3, [[111, 112]] * 3, [[101, 102]] * 3]], "s32")])

# ---- put_slice and slice with dynamic starts: nx/lib/nx.ex:14421-14464, 14080-14103 ---------------------
case("put_slice 1d", "nx/lib/nx.ex:14424-14429", lambda t, s: nx.put_slice(t, [2], s),
     [([0, 1, 2, 3, 4], "s32"), ([5, 6], "s32")], [([0, 1, 5, 6, 4], "s32")])
case("put_slice 2d", "nx/lib/nx.ex:14431-14439", lambda t, s: nx.put_slice(t, [0, 1], s),
     [([[1, 2, 3], [4, 5, 6]], "s32"), ([[7, 8], [9, 10]], "s32")], [([[1, 7, 8], [4, 9, 10]], "s32")])
case("put_slice dynamic starts, merged type", "nx/lib/nx.ex:14443-14451",
     lambda t, a, b, s: nx.put_slice(t, [a, b], s),
     [([[1, 2, 3], [4, 5, 6]], "s32"), (0, "s32"), (1, "s32"), ([[10.0, 11.0]], "f32")],
     [([[1.0, 10.0, 11.0], [4.0, 5.0, 6.0]], "f32")])
case("put_slice clips the start", "nx/lib/nx.ex:14456-14464", lambda t, a, s: nx.put_slice(t, [a, 1], s),
     [([[1, 2, 3], [4, 5, 6]], "s32"), (1, "s32"), ([[7, 8], [9, 10]], "s32")], [([[1, 7, 8], [4, 9, 10]], "s32")])
case("slice dynamic starts with strides", "nx/lib/nx.ex:14080-14103",
     lambda t, a, b: nx.slice(t, [a, b], [6, 7], strides=[5, 3]),
     [([[0.0] * 7] * 2 + [[1.0] * 7] * 4, "f32"), (0, "s32"), (0, "s32")], [([[0.0] * 3, [1.0] * 3], "f32")])
case("slice dynamic starts", "nx/lib/nx.ex:14077-14084", lambda t, a, b: nx.slice(t, [a, b], [1, 1]),
     [([[1, 2, 3], [4, 5, 6]], "s32"), (1, "s32"), (2, "s32")], [([[6]], "s32")])
case("slice dynamic start is clipped", "nx/lib/nx.ex:14105-14125", lambda t, a: nx.slice(t, [a, 0], [2, 2]),
     [([[1, 2], [3, 4], [5, 6]], "s32"), (2, "s32")], [([[3, 4], [5, 6]], "s32")])

# ---- pad / reverse / take_along_axis: exla/test/exla/defn/expr_test.exs:3095-3182, 3498-3540; nx/lib/nx.ex doctests ----
case("pad vector", "exla/test/exla/defn/expr_test.exs:3108-3110", lambda t: nx.pad(t, 0, [(1, 1, 0)]),
     [([1, 2, 3], "s32")], [([0, 1, 2, 3, 0], "s32")])
case("pad matrix", "exla/test/exla/defn/expr_test.exs:3112-3117", lambda t: nx.pad(t, 0, [(1, 1, 0), (1, 1, 0)]),
     [([[1, 2, 3], [4, 5, 6]], "s32")], [([[0, 0, 0, 0, 0], [0, 1, 2, 3, 0], [0, 4, 5, 6, 0], [0, 0, 0, 0, 0]], "s32")])
_PADDED = [[[0.0] * 3] * 3, [[0.0] * 3, [1.0, 2.0, 0.0], [3.0, 4.0, 0.0]], [[0.0] * 3, [5.0, 6.0, 0.0], [7.0, 8.0, 0.0]],
           [[0.0] * 3] * 3, [[0.0] * 3] * 3]
case("pad tensor, float pad value on integers", "exla/test/exla/defn/expr_test.exs:3119-3156",
     lambda t: nx.pad(t, 0.0, [(1, 2, 0), (1, 0, 0), (0, 1, 0)]), [([[[1, 2], [3, 4]], [[5, 6], [7, 8]]], "s32")], [(_PADDED, "f32")])
case("pad interior", "nx/lib/nx.ex:4055-4063", lambda t: nx.pad(t, 0, [(0, 0, 1), (0, 0, 1)]),
     [([[1, 2, 3], [4, 5, 6]], "s32")], [([[1, 0, 2, 0, 3], [0, 0, 0, 0, 0], [4, 0, 5, 0, 6]], "s32")])
case("pad negative vector", "exla/test/exla/defn/expr_test.exs:3159-3162", lambda t: nx.pad(t, 0.0, [(-1, -1, 0)]),
     [([1.0, 1.0, 2.0, 3.0, 0.0], "f32")], [([1.0, 2.0, 3.0], "f32")])
case("pad negative matrix", "exla/test/exla/defn/expr_test.exs:3164-3167", lambda t: nx.pad(t, 0, [(0, 0, 0), (-1, 1, 0)]),
     [([[0, 1, 2, 3], [0, 4, 5, 6]], "s32")], [([[1, 2, 3, 0], [4, 5, 6, 0]], "s32")])
case("pad negative tensor", "exla/test/exla/defn/expr_test.exs:3169-3180",
     lambda t: nx.pad(t, 0, [(-1, 0, 0), (-1, -1, 0), (0, -1, 0)]),
     [([[[0, 0, 0]] * 4, [[0, 0, 0], [1, 2, 0], [3, 4, 0], [0, 0, 0]], [[0, 0, 0], [5, 6, 0], [7, 8, 0], [0, 0, 0]]], "s32")],
     [([[[1, 2], [3, 4]], [[5, 6], [7, 8]]], "s32")])
case("reverse all dims", "exla/test/exla/defn/expr_test.exs:3506-3507", lambda t: nx.reverse(t),
     [([[0, 1, 2, 3], [4, 5, 6, 7]], "s32")], [([[7, 6, 5, 4], [3, 2, 1, 0]], "s32")])
case("reverse one dim", "exla/test/exla/defn/expr_test.exs:3529-3530", lambda t: nx.reverse(t, axes=[1]),
     [([[0, 1, 2], [3, 4, 5]], "s32")], [([[2, 1, 0], [5, 4, 3]], "s32")])
case("take_along_axis 1", "nx/lib/nx.ex:14839-14847", lambda t, i: nx.take_along_axis(t, i, axis=1),
     [([[1, 2, 3], [4, 5, 6]], "s32"), ([[0, 0, 2, 2, 1, 1], [2, 2, 1, 1, 0, 0]], "s32")],
     [([[1, 1, 3, 3, 2, 2], [6, 6, 5, 5, 4, 4]], "s32")])
case("take_along_axis 0", "nx/lib/nx.ex:14849-14858", lambda t, i: nx.take_along_axis(t, i, axis=0),
     [([[1, 2, 3], [4, 5, 6]], "s32"), ([[0, 1, 1], [1, 0, 0], [0, 1, 0]], "s32")],
     [([[1, 5, 6], [4, 2, 3], [1, 5, 3]], "s32")])
case("stack", "nx/lib/nx.ex stack doctest", lambda a, b: nx.stack([a, b], axis=1),
     [([1, 2, 3], "s32"), ([4, 5, 6], "s32")], [([[1, 4], [2, 5], [3, 6]], "s32")])

# ---- window reductions: exla/test/exla/defn/expr_test.exs:2309-2600 -------------------------------------
W3 = [[[1, 2, 3], [4, 5, 6]], [[1, 2, 3], [4, 5, 6]]]
WF = [[[4.0, 2.0, 3.0], [2.0, 5.0, 6.5]], [[1.2, 2.2, 3.2], [4.0, 5.0, 6.2]]]
_P2 = dict(strides=[1, 2, 3], padding=[(0, 1), (2, 0), (1, 1)])
_P3 = dict(strides=[2, 1, 1], padding=[(1, 1), (0, 0), (1, 1)])
case("window_sum", "exla/test/exla/defn/expr_test.exs:2323-2326", lambda t: nx.window_sum(t, (1, 2, 1)), [(W3, "s32")],
     [([[[5, 7, 9]], [[5, 7, 9]]], "s32")])
case("window_sum strides + padding", "exla/test/exla/defn/expr_test.exs:2328-2331", lambda t: nx.window_sum(t, (2, 2, 1), **_P2),
     [(W3, "s32")], [([[[0, 0], [0, 18]], [[0, 0], [0, 9]]], "s32")])
case("window_sum float padding", "exla/test/exla/defn/expr_test.exs:2333-2341", lambda t: nx.window_sum(t, (2, 1, 1), **_P3),
     [(WF, "f32")], [([[[0.0, 4.0, 2.0, 3.0, 0.0], [0.0, 2.0, 5.0, 6.5, 0.0]], [[0.0, 1.2, 2.2, 3.2, 0.0], [0.0, 4.0, 5.0, 6.2, 0.0]]], "f32")])
case("window_max", "exla/test/exla/defn/expr_test.exs:2428-2431", lambda t: nx.window_max(t, (1, 2, 1)), [(W3, "s32")],
     [([[[4, 5, 6]], [[4, 5, 6]]], "s32")])
_MIN = -2147483648
case("window_max strides + padding", "exla/test/exla/defn/expr_test.exs:2433-2445", lambda t: nx.window_max(t, (2, 2, 1), **_P2),
     [(W3, "s32")], [([[[_MIN, _MIN], [_MIN, 6]], [[_MIN, _MIN], [_MIN, 6]]], "s32")])
case("window_max float padding", "exla/test/exla/defn/expr_test.exs:2447-2461", lambda t: nx.window_max(t, (2, 1, 1), **_P3),
     [(WF, "f32")], [([[[-INF, 4.0, 2.0, 3.0, -INF], [-INF, 2.0, 5.0, 6.5, -INF]], [[-INF, 1.2, 2.2, 3.2, -INF], [-INF, 4.0, 5.0, 6.2, -INF]]], "f32")])
case("window_min", "exla/test/exla/defn/expr_test.exs:2493-2496", lambda t: nx.window_min(t, (1, 2, 1)), [(W3, "s32")],
     [([[[1, 2, 3]], [[1, 2, 3]]], "s32")])
case("window_product", "exla/test/exla/defn/expr_test.exs:2563-2566", lambda t: nx.window_product(t, (1, 2, 1)), [(W3, "s32")],
     [([[[4, 10, 18]], [[4, 10, 18]]], "s32")])
case("window_mean", "nx/lib/nx.ex:11235-11250", lambda t: nx.window_mean(t, (1, 2, 1)), [(W3, "s32")],
     [([[[2.5, 3.5, 4.5]], [[2.5, 3.5, 4.5]]], "f32")])

# ---- conv: nx/lib/nx.ex:13684-13740 (doctests) ---------------------------------------------------------
_I33 = [[[[0, 1, 2], [3, 4, 5], [6, 7, 8]]]]
case("conv 1x1 kernels", "nx/lib/nx.ex:13684-13713", lambda a, b: nx.conv(a, b, strides=[1, 1]),
     [(_I33, "s32"), ([[[[0]]], [[[1]]], [[[2]]], [[[3]]]], "s32")],
     [([[[[0.0] * 3] * 3, [[0.0, 1.0, 2.0], [3.0, 4.0, 5.0], [6.0, 7.0, 8.0]], [[0.0, 2.0, 4.0], [6.0, 8.0, 10.0], [12.0, 14.0, 16.0]],
         [[0.0, 3.0, 6.0], [9.0, 12.0, 15.0], [18.0, 21.0, 24.0]]]], "f32")])
case("conv strides, same padding, kernel dilation", "nx/lib/nx.ex:13715-13740",
     lambda a, b: nx.conv(a, b, strides=2, padding="same", kernel_dilation=[2, 1]),
     [(_I33, "s32"), ([[[[0], [1]]], [[[2], [3]]], [[[4], [5]]], [[[6], [7]]]], "s32")],
     [([[[[3.0, 5.0], [0.0, 0.0]], [[9.0, 15.0], [6.0, 10.0]], [[15.0, 25.0], [12.0, 20.0]], [[21.0, 35.0], [18.0, 30.0]]]], "f32")])

# ---- sort / argsort / top_k: nx/lib/nx.ex:15538-15689, 15730-15800, 15880-15945 -------------------------
_S23 = [[3, 1, 7], [2, 5, 4]]
_S233 = [[[4, 9, 8], [2, 1, 3], [2, 0, 2]], [[1, 5, 2], [2, 5, 3], [5, 1, 4]]]
case("sort 1d", "nx/lib/nx.ex:15538-15542", lambda t: nx.sort(t), [([16, 23, 42, 4, 8, 15], "s32")], [([4, 8, 15, 16, 23, 42], "s32")])
case("sort axis 0", "nx/lib/nx.ex:15544-15552", lambda t: nx.sort(t, axis=0), [(_S23, "s32")], [([[2, 1, 4], [3, 5, 7]], "s32")])
case("sort axis 1", "nx/lib/nx.ex:15554-15562", lambda t: nx.sort(t, axis=1), [(_S23, "s32")], [([[1, 3, 7], [2, 4, 5]], "s32")])
case("sort rank 3 axis 0", "nx/lib/nx.ex:15627-15642", lambda t: nx.sort(t, axis=0), [(_S233, "s32")],
     [([[[1, 5, 2], [2, 1, 3], [2, 0, 2]], [[4, 9, 8], [2, 5, 3], [5, 1, 4]]], "s32")])
case("sort rank 3 axis 1", "nx/lib/nx.ex:15643-15658", lambda t: nx.sort(t, axis=1), [(_S233, "s32")],
     [([[[2, 0, 2], [2, 1, 3], [4, 9, 8]], [[1, 1, 2], [2, 5, 3], [5, 5, 4]]], "s32")])
case("sort rank 3 axis 2", "nx/lib/nx.ex:15659-15674", lambda t: nx.sort(t, axis=2), [(_S233, "s32")],
     [([[[4, 8, 9], [1, 2, 3], [0, 2, 2]], [[1, 2, 5], [2, 3, 5], [1, 4, 5]]], "s32")])
case("sort NaN and infinities", "nx/lib/nx.ex:15679-15684", lambda t: nx.sort(t), [([NAN, -INF, 0.0, INF], "f32")],
     [([-INF, 0.0, INF, NAN], "f32")])
case("sort desc NaN first", "nx/lib/nx.ex:15685-15689", lambda t: nx.sort(t, direction="desc"), [([NAN, -INF, 0.0, INF], "f32")],
     [([NAN, INF, 0.0, -INF], "f32")])
case("argsort 1d", "nx/lib/nx.ex argsort doctest", lambda t: nx.argsort(t), [([16, 23, 42, 4, 8, 15], "s32")], [([3, 4, 5, 0, 1, 2], "s32")])
case("argsort ties are stable", "nx/lib/nx.ex argsort stable: true", lambda t: nx.argsort(t, axis=1, direction="desc", stable=True),
     [([[1, 3, 3, 1], [2, 2, 5, 2]], "s32")], [([[1, 2, 0, 3], [2, 0, 1, 3]], "s32")])
case("top_k", "nx/lib/nx.ex top_k doctest", lambda t: nx.top_k(t, k=2), [([[1, 5, 3], [9, 2, 7]], "s32")],
     [([[5, 3], [9, 7]], "s32"), ([[1, 2], [0, 2]], "s32")])

# ---- indexed_add / indexed_put: exla/test/exla/defn/expr_test.exs:1776-1920, nx/lib/nx.ex:8166-8440 ----
_Z234 = [[[0] * 4 for _ in range(3)] for _ in range(2)]
case("indexed_add multi-dim", "exla/test/exla/defn/expr_test.exs:1781-1822", lambda t, i, u: nx.indexed_add(t, i, u),
     [(_Z234, "s32"), ([[0, 0, 0], [0, 0, 1], [0, 0, 0], [0, 1, 1], [1, 2, 2], [1, 2, 3], [1, 0, 3]], "s32"), ([1, 1, -1, 2, -1, 3, 4], "s32")],
     [([[[0, 1, 0, 0], [0, 2, 0, 0], [0, 0, 0, 0]], [[0, 0, 0, 4], [0, 0, 0, 0], [0, 0, -1, 3]]], "s32")])
case("indexed_add s32 + s32", "exla/test/exla/defn/expr_test.exs:1825-1829", lambda t, i, u: nx.indexed_add(t, i, u),
     [([0], "s32"), ([[0]], "s32"), ([1], "s32")], [([1], "s32")])
case("indexed_add s32 + f32", "exla/test/exla/defn/expr_test.exs:1831-1835", lambda t, i, u: nx.indexed_add(t, i, u),
     [([0], "s32"), ([[0]], "s32"), ([1.0], "f32")], [([1.0], "f32")])
case("indexed_add f32 + s32", "exla/test/exla/defn/expr_test.exs:1837-1841", lambda t, i, u: nx.indexed_add(t, i, u),
     [([0.0], "f32"), ([[0]], "s32"), ([1], "s32")], [([1.0], "f32")])
case("indexed_add f64 + f32", "exla/test/exla/defn/expr_test.exs:1843-1847", lambda t, i, u: nx.indexed_add(t, i, u),
     [([0.0], "f64"), ([[0]], "s32"), ([1.0], "f32")], [([1.0], "f64")])
case("indexed_add repeated index accumulates", "nx/lib/nx.ex:8214-8218", lambda t, i, u: nx.indexed_add(t, i, u),
     [([1.0], "f32"), ([[0], [0]], "s32"), ([1, 1], "s32")], [([3.0], "f32")])
case("indexed_add s32 + s64", "nx/lib/nx.ex:8226-8230", lambda t, i, u: nx.indexed_add(t, i, u),
     [([1], "s32"), ([[0], [0]], "s32"), ([1, 1], "s64")], [([3], "s64")])
case("indexed_add rank-1 index, scalar update", "nx/lib/nx.ex:8182-8189", lambda t, i: nx.indexed_add(t, i, 8),
     [([[1], [2]], "s32"), ([1, 0], "s32")], [([[1], [10]], "s32")])
case("indexed_add iota {1,2,3}", "nx/lib/nx.ex:8193-8212", lambda t, i, u: nx.indexed_add(t, i, u),
     [([[[0, 1, 2], [3, 4, 5]]], "s32"), ([[0, 0, 0], [0, 1, 1], [0, 0, 0], [0, 0, 2], [0, 1, 2]], "s32"), ([1, 3, 1, -2, 5], "s32")],
     [([[[2, 1, 0], [3, 7, 10]]], "s32")])
case("indexed_put multi-dim", "exla/test/exla/defn/expr_test.exs:1859-1896", lambda t, i, u: nx.indexed_put(t, i, u),
     [(_Z234, "s32"), ([[0, 0, 1], [0, 0, 0], [0, 1, 1], [1, 2, 2], [1, 2, 3], [1, 0, 3]], "s32"), ([1, -1, 2, -1, 3, 4], "s32")],
     [([[[-1, 1, 0, 0], [0, 2, 0, 0], [0, 0, 0, 0]], [[0, 0, 0, 4], [0, 0, 0, 0], [0, 0, -1, 3]]], "s32")])
case("indexed_put s32 <- f32", "exla/test/exla/defn/expr_test.exs:1905-1909", lambda t, i, u: nx.indexed_put(t, i, u),
     [([0], "s32"), ([[0]], "s32"), ([1.0], "f32")], [([1.0], "f32")])
case("indexed_put f64 <- f32", "exla/test/exla/defn/expr_test.exs:1917-1921", lambda t, i, u: nx.indexed_put(t, i, u),
     [([0.0], "f64"), ([[0]], "s32"), ([1.0], "f32")], [([1.0], "f64")])
case("indexed_put rows on a given dimension", "nx/lib/nx.ex:8348-8370", lambda t, i, u: nx.indexed_put(t, i, u),
     [([[[0, 1], [2, 3], [4, 5]]], "s32"), ([[0, 0], [0, 2]], "s32"), ([[0, 10], [40, 50]], "s32")],
     [([[[0, 10], [2, 3], [40, 50]]], "s32")])
case("indexed_put axes [0, 2]", "nx/lib/nx.ex:8376-8404", lambda t, i, u: nx.indexed_put(t, i, u, axes=[0, 2]),
     [([[[0, 1, 2], [3, 4, 5]]], "s32"), ([[0, 0], [0, 2]], "s32"), ([[0, 30], [20, 50]], "s32")],
     [([[[0, 1, 20], [30, 4, 50]]], "s32")])
case("indexed_put rank-1 index, scalar update", "nx/lib/nx.ex:8306-8313", lambda t, i: nx.indexed_put(t, i, 10),
     [([[1], [2]], "s32"), ([1, 0], "s32")], [([[1], [10]], "s32")])

# ---- element-wise binary operators: doctests of nx/lib/nx.ex -----------------------------------------
case("remainder tensor, scalar", "nx/lib/nx.ex:6407-6411", lambda t: nx.remainder(t, 2), [([1, 2, 3], "s32")], [([1, 0, 1], "s32")])
case("remainder scalar, f32 tensor", "nx/lib/nx.ex:6413-6417", lambda t: nx.remainder(2, t), [([1.0, 2.0, 3.0], "f32")], [([0.0, 0.0, 2.0], "f32")])
case("remainder broadcast", "nx/lib/nx.ex:6421-6430", lambda a, b: nx.remainder(a, b), [([[10], [20]], "s32"), ([[3, 4]], "s32")],
     [([[1, 2], [2, 0]], "s32")])
case("remainder s8 by u8 keeps the dividend's sign", "nx/lib/nx.ex:6440-6451",
     lambda a, b: (nx.remainder(a, b), nx.remainder(nx.add(a, nx.tensor(20, "s8")), b)), [(-11, "s8"), (10, "u8")], [(-1, "s16"), (9, "s16")])
case("remainder u8", "nx/lib/nx.ex:6452-6462",
     lambda a, b: (nx.remainder(a, b), nx.remainder(nx.add(a, nx.tensor(20, "u8")), b)), [(9, "u8"), (10, "u8")], [(9, "u8"), (9, "u8")])
case("quotient tensor, scalar", "nx/lib/nx.ex:6593-6597", lambda t: nx.quotient(t, 2), [([2, 4, 5], "s32")], [([1, 2, 2], "s32")])
case("quotient scalar, tensor", "nx/lib/nx.ex:6599-6603", lambda t: nx.quotient(10, t), [([1, 2, 3], "s32")], [([10, 5, 3], "s32")])
case("quotient broadcast s8", "nx/lib/nx.ex:6618-6627", lambda a, b: nx.quotient(a, b), [([[10, 20]], "s8"), ([[1], [2]], "s8")],
     [([[10, 20], [5, 10]], "s8")])
case("quotient u8 by u32", "nx/lib/nx.ex:6629-6638", lambda a, b: nx.quotient(a, b), [([[10, 20]], "u8"), ([[1], [2]], "u32")],
     [([[10, 20], [5, 10]], "u32")])
case("pow tensor, scalar", "nx/lib/nx.ex:6357-6361", lambda t: nx.pow(t, 2), [([1, 2, 3], "s32")], [([1, 4, 9], "s32")])
case("pow scalar, f32 tensor", "nx/lib/nx.ex:6363-6367", lambda t: nx.pow(2, t), [([1.0, 2.0, 3.0], "f32")], [([2.0, 4.0, 8.0], "f32")],
     exact=False)
case("pow broadcast", "nx/lib/nx.ex:6371-6379", lambda a, b: nx.pow(a, b), [([[2], [3]], "s32"), ([[4, 5]], "s32")],
     [([[16, 32], [81, 243]], "s32")])
case("atan2 tensor, scalar", "nx/lib/nx.ex:6668-6672", lambda t: nx.atan2(t, 1), [([1, 2, 3], "s32")],
     [([0.7853982, 1.1071488, 1.2490457], "f32")], exact=False)
case("atan2 scalar, tensor", "nx/lib/nx.ex:6674-6678", lambda t: nx.atan2(1, t), [([1.0, 2.0, 3.0], "f32")],
     [([0.7853982, 0.4636476, 0.32175055], "f32")], exact=False)
case("atan2 signed zeros f64", "nx/lib/nx.ex:6682-6692", lambda a, b: nx.atan2(a, b), [([[-0.0], [0.0]], "f64"), ([-0.0, 0.0], "f64")],
     [([[-3.141592653589793, -0.0], [3.141592653589793, 0.0]], "f64")], exact=False)
case("max broadcast s8", "nx/lib/nx.ex:6745-6754", lambda a, b: nx.max(a, b), [([[1], [2]], "s8"), ([[10, 20]], "s8")],
     [([[10, 20], [10, 20]], "s8")])
case("max broadcast f32", "nx/lib/nx.ex:6756-6765", lambda a, b: nx.max(a, b), [([[1], [2]], "f32"), ([[10, 20]], "f32")],
     [([[10.0, 20.0], [10.0, 20.0]], "f32")])
case("bitwise_and tensor, scalar", "nx/lib/nx.ex:6883-6887", lambda t: nx.bitwise_and(t, 1), [([0, 1, 2], "s32")], [([0, 1, 0], "s32")])
case("bitwise_and negative", "nx/lib/nx.ex:6889-6893", lambda t: nx.bitwise_and(t, -1), [([0, -1, -2], "s32")], [([0, -1, -2], "s32")])
case("bitwise_and tensors", "nx/lib/nx.ex:6897-6901", lambda a, b: nx.bitwise_and(a, b), [([0, 0, 1, 1], "s32"), ([0, 1, 0, 1], "s32")],
     [([0, 0, 0, 1], "s32")])
case("bitwise_xor tensor, scalar", "nx/lib/nx.ex:6988-6992", lambda t: nx.bitwise_xor(t, 2), [([1, 2, 3], "s32")], [([3, 0, 1], "s32")])
case("bitwise_xor negative", "nx/lib/nx.ex:6994-6998", lambda t: nx.bitwise_xor(t, 2), [([-1, -2, -3], "s32")], [([-3, -4, -1], "s32")])
case("left_shift tensor, scalar", "nx/lib/nx.ex:7045-7049", lambda t: nx.left_shift(t, 2), [([1, 2, 3], "s32")], [([4, 8, 12], "s32")])
case("left_shift tensors", "nx/lib/nx.ex:7053-7059", lambda a, b: nx.left_shift(a, b), [([1, 1, -1, -1], "s32"), ([1, 2, 3, 4], "s32")],
     [([2, 4, -8, -16], "s32")])
case("right_shift tensor, scalar", "nx/lib/nx.ex:7103-7107", lambda t: nx.right_shift(t, 2), [([2, 4, 8], "s32")], [([0, 1, 2], "s32")])
case("right_shift tensors (arithmetic for signed)", "nx/lib/nx.ex:7111-7117", lambda a, b: nx.right_shift(a, b),
     [([16, 32, -64, -128], "s32"), ([1, 2, 3, 4], "s32")], [([8, 8, -8, -8], "s32")])
case("logical_and scalar, tensor", "nx/lib/nx.ex:7196-7200", lambda t: nx.logical_and(1, t), [([-1, 0, 1], "s32")], [([1, 0, 1], "u8")])
case("logical_and broadcast, f32 with s32", "nx/lib/nx.ex:7214-7225", lambda a, b: nx.logical_and(a, b),
     [([-1.0, 0.0, 1.0], "f32"), ([[-1], [0], [1]], "s32")], [([[1, 0, 1], [0, 0, 0], [1, 0, 1]], "u8")])
case("logical_xor scalar, tensor", "nx/lib/nx.ex:7287-7291", lambda t: nx.logical_xor(0, t), [([-1, 0, 1], "s32")], [([1, 0, 1], "u8")])
case("logical_xor broadcast", "nx/lib/nx.ex:7293-7304", lambda a, b: nx.logical_xor(a, b),
     [([-1, 0, 1], "s32"), ([[-1], [0], [1]], "s32")], [([[0, 1, 0], [1, 0, 1], [0, 1, 0]], "u8")])

# ---- clip: nx/lib/nx.ex:13906-13955 --------------------------------------------------------------------
_T23 = [[1, 2, 3], [4, 5, 6]]
case("clip s32", "nx/lib/nx.ex:13906-13914", lambda t: nx.clip(t, 2, 4), [(_T23, "s32")], [([[2, 2, 3], [4, 4, 4]], "s32")])
case("clip s32 by a float bound", "nx/lib/nx.ex:13916-13924", lambda t: nx.clip(t, 2.0, 3), [(_T23, "s32")],
     [([[2.0, 2.0, 3.0], [3.0, 3.0, 3.0]], "f32")])
case("clip f32", "nx/lib/nx.ex:13936-13944", lambda t: nx.clip(t, 2, 6.0), [(_T23, "f32")], [([[2.0, 2.0, 3.0], [4.0, 5.0, 6.0]], "f32")])
case("clip f32 integer bounds", "nx/lib/nx.ex:13946-13954", lambda t: nx.clip(t, 1, 4), [(_T23, "f32")],
     [([[1.0, 2.0, 3.0], [4.0, 4.0, 4.0]], "f32")])

# ---- reduce_min, product, all, any: nx/lib/nx.ex doctests ------------------------------------------------
case("reduce_min", "nx/lib/nx.ex:10530-10534", lambda t: nx.reduce_min(t), [([1, 2, 3], "s32")], [(1, "s32")])
case("reduce_min axis 0", "nx/lib/nx.ex:10538-10543", lambda t: nx.reduce_min(t, axes=[0]), [([[3, 1, 4], [2, 1, 1]], "s32")], [([2, 1, 1], "s32")])
case("reduce_min axis 1", "nx/lib/nx.ex:10545-10550", lambda t: nx.reduce_min(t, axes=[1]), [([[3, 1, 4], [2, 1, 1]], "s32")], [([1, 1], "s32")])
_M222 = [[[1, 2], [4, 5]], [[2, 4], [3, 8]]]
case("reduce_min axes 0,2", "nx/lib/nx.ex:10552-10557", lambda t: nx.reduce_min(t, axes=[0, 2]), [(_M222, "s32")], [([1, 3], "s32")])
case("reduce_min axes 0,2 keep", "nx/lib/nx.ex:10561-10572", lambda t: nx.reduce_min(t, axes=[0, 2], keep_axes=True), [(_M222, "s32")],
     [([[[1], [3]]], "s32")])
case("product", "nx/lib/nx.ex:10290-10294", lambda t: nx.product(t), [([1, 2, 3], "s32")], [(6, "s32")])
case("product f32", "nx/lib/nx.ex:10296-10300", lambda t: nx.product(t), [([[1.0, 2.0], [3.0, 4.0]], "f32")], [(24.0, "f32")])
case("product u8 -> u32", "nx/lib/nx.ex:10305-10309", lambda t: nx.product(t), [([[10, 20], [30, 40]], "u8")], [(240000, "u32")])
case("product s8 -> s32", "nx/lib/nx.ex:10311-10315", lambda t: nx.product(t), [([[10, 20], [30, 40]], "s8")], [(240000, "s32")])
_I223 = [[[0, 1, 2], [3, 4, 5]], [[6, 7, 8], [9, 10, 11]]]
case("product axis 0", "nx/lib/nx.ex:10327-10335", lambda t: nx.product(t, axes=[0]), [(_I223, "s32")], [([[0, 7, 16], [27, 40, 55]], "s32")])
case("product axis 1", "nx/lib/nx.ex:10336-10343", lambda t: nx.product(t, axes=[1]), [(_I223, "s32")], [([[0, 4, 10], [54, 70, 88]], "s32")])
case("product axes 0,2", "nx/lib/nx.ex:10344-10348", lambda t: nx.product(t, axes=[0, 2]), [(_I223, "s32")], [([0, 59400], "s32")])
case("all", "nx/lib/nx.ex:9155-9159", lambda t: nx.all(t), [([0, 1, 2], "s32")], [(0, "u8")])
case("all axis 0", "nx/lib/nx.ex:9161-9165", lambda t: nx.all(t, axes=[0]), [([[-1, 0, 1], [2, 3, 4]], "s32")], [([1, 0, 1], "u8")])
case("all axis 1", "nx/lib/nx.ex:9167-9171", lambda t: nx.all(t, axes=[1]), [([[-1, 0, 1], [2, 3, 4]], "s32")], [([0, 1], "u8")])
case("all axis 1 keep", "nx/lib/nx.ex:9175-9182", lambda t: nx.all(t, axes=[1], keep_axes=True), [([[-1, 0, 1], [2, 3, 4]], "s32")],
     [([[0], [1]], "u8")])
case("any", "nx/lib/nx.ex:9228-9232", lambda t: nx.any(t), [([0, 1, 2], "s32")], [(1, "u8")])
case("any axis 0", "nx/lib/nx.ex:9234-9238", lambda t: nx.any(t, axes=[0]), [([[0, 1, 0], [0, 1, 2]], "s32")], [([0, 1, 1], "u8")])
case("any axis 1", "nx/lib/nx.ex:9240-9244", lambda t: nx.any(t, axes=[1]), [([[0, 1, 0], [0, 1, 2]], "s32")], [([1, 1], "u8")])
case("any axis 1 keep", "nx/lib/nx.ex:9248-9255", lambda t: nx.any(t, axes=[1], keep_axes=True), [([[0, 1, 0], [0, 1, 2]], "s32")],
     [([[1], [1]], "u8")])

# ---- element-wise unary operators and predicates: doctests of nx/lib/nx.ex --------------------------------
case("sign", "nx/lib/nx.ex:8719-8723", lambda t: nx.sign(t), [([-2, -1, 0, 1, 2], "s32")], [([-1, -1, 0, 1, 1], "s32")])
case("abs", "nx/lib/nx.ex:8738-8742", lambda t: nx.abs(t), [([-2, -1, 0, 1, 2], "s32")], [([2, 1, 0, 1, 2], "s32")])
case("negate s32", "nx/lib/nx.ex:8681-8685", lambda t: nx.negate(t), [([-1, 0, 1], "s32")], [([1, 0, -1], "s32")])
case("negate f32", "nx/lib/nx.ex:8687-8691", lambda t: nx.negate(t), [([1.0, 2.0, 3.0], "f32")], [([-1.0, -2.0, -3.0], "f32")])
case("negate u8 wraps", "nx/lib/nx.ex:8695-8699", lambda t: nx.negate(t), [([0, 1, 2], "u8")], [([0, 255, 254], "u8")])
case("bitwise_not s8", "nx/lib/nx.ex:8961-8965", lambda t: nx.bitwise_not(t), [([-1, 0, 1], "s8")], [([0, -1, -2], "s8")])
case("bitwise_not u8", "nx/lib/nx.ex:8967-8971", lambda t: nx.bitwise_not(t), [([0, 1, 254, 255], "u8")], [([255, 254, 1, 0], "u8")])
case("population_count s32", "nx/lib/nx.ex:9003-9007", lambda t: nx.population_count(t), [([0, 1, 254, 255], "s32")], [([0, 1, 7, 8], "s32")])
case("population_count s8", "nx/lib/nx.ex:9009-9013", lambda t: nx.population_count(t), [([0, 1, 126, 127, -1, -127, -128], "s8")],
     [([0, 1, 6, 7, 8, 2, 1], "s8")])
case("count_leading_zeros s32", "nx/lib/nx.ex:9045-9049", lambda t: nx.count_leading_zeros(t), [([0, 0xF, 0xFF, 0xFFFF], "s32")],
     [([32, 28, 24, 16], "s32")])
case("count_leading_zeros s64", "nx/lib/nx.ex:9057-9061", lambda t: nx.count_leading_zeros(t), [([0, 0xF, 0xFF, 0xFFFF], "s64")],
     [([64, 60, 56, 48], "s64")])
case("count_leading_zeros s16", "nx/lib/nx.ex:9063-9067", lambda t: nx.count_leading_zeros(t), [([0, 0xF, 0xFF, 0xFFFF], "s16")],
     [([16, 12, 8, 0], "s16")])
case("is_nan", "nx/lib/nx.ex:8609-8613", lambda t: nx.is_nan(t), [([NAN, 1, 0], "f32")], [([1, 0, 0], "u8")])
case("is_infinity", "nx/lib/nx.ex:8642-8646", lambda t: nx.is_infinity(t), [([INF, NAN, -INF, 1, 0], "f32")], [([1, 0, 1, 0, 0], "u8")])
case("less tensors", "nx/lib/nx.ex:7519-7523", lambda a, b: nx.less(a, b), [([1, 2, 1], "s32"), ([1, 2, 2], "s32")], [([0, 0, 1], "u8")])
case("less f32 with s32, broadcast", "nx/lib/nx.ex:7525-7532", lambda a, b: nx.less(a, b),
     [([[1.0, 2.0, 3.0], [4.0, 2.0, 1.0]], "f32"), ([1, 2, 3], "s32")], [([[0, 0, 0], [0, 0, 1]], "u8")])

# ---- shape operators: doctests of nx/lib/nx.ex -----------------------------------------------------------
_I234 = [[[0, 1, 2, 3], [4, 5, 6, 7], [8, 9, 10, 11]], [[12, 13, 14, 15], [16, 17, 18, 19], [20, 21, 22, 23]]]
_I234_T = [[[0, 12], [4, 16], [8, 20]], [[1, 13], [5, 17], [9, 21]], [[2, 14], [6, 18], [10, 22]], [[3, 15], [7, 19], [11, 23]]]
case("transpose default (reverse axes)", "nx/lib/nx.ex:13283-13308", lambda t: nx.transpose(t), [(_I234, "s32")], [(_I234_T, "s32")])
case("transpose axes [2,1,0]", "nx/lib/nx.ex:13316-13341", lambda t: nx.transpose(t, axes=[2, 1, 0]), [(_I234, "s32")], [(_I234_T, "s32")])
case("broadcast column to the shape of a tensor", "nx/lib/nx.ex:3792-3799", lambda a: nx.broadcast(a, (2, 2)), [([[1], [2]], "s32")],
     [([[1, 1], [2, 2]], "s32")])
case("broadcast row", "nx/lib/nx.ex:3801-3808", lambda a: nx.broadcast(a, (2, 2)), [([[1, 2]], "s32")], [([[1, 2], [1, 2]], "s32")])
case("broadcast with axes", "nx/lib/nx.ex:3838-3847", lambda t: nx.broadcast(t, (3, 2), axes=[0]), [([1, 2, 3], "s32")],
     [([[1, 1], [2, 2], [3, 3]], "s32")])
case("concatenate merges types", "nx/lib/nx.ex:15241-15264", lambda a, b, c: nx.concatenate([a, b, c], axis=0),
     [([[[0, 1], [2, 3]], [[4, 5], [6, 7]]], "f32"), ([[[0, 1], [2, 3]]], "u8"), ([[[0, 1], [2, 3]]], "s64")],
     [([[[0.0, 1.0], [2.0, 3.0]], [[4.0, 5.0], [6.0, 7.0]], [[0.0, 1.0], [2.0, 3.0]], [[0.0, 1.0], [2.0, 3.0]]], "f32")])
case("concatenate axis 1", "nx/lib/nx.ex:15269-15285", lambda a, b, c: nx.concatenate([a, b, c], axis=1),
     [([[[0, 1], [2, 3], [4, 5]]], "s32"), ([[[0, 1]]], "s32"), ([[[0, 1], [2, 3]]], "s32")],
     [([[[0, 1], [2, 3], [4, 5], [0, 1], [0, 1], [2, 3]]], "s32")])
case("iota over all axes / along an axis", "nx/lib/nx.ex:1118-1145",
     lambda t: (nx.add(nx.iota((3, 2, 3)), t), nx.add(nx.iota((3, 3), axis=1), t)), [(0, "s32")],
     [([[[0, 1, 2], [3, 4, 5]], [[6, 7, 8], [9, 10, 11]], [[12, 13, 14], [15, 16, 17]]], "s32"), ([[0, 1, 2], [0, 1, 2], [0, 1, 2]], "s32")])

# ---- mean, logical_not, comparisons, slice_along_axis: doctests of nx/lib/nx.ex ----------------------------
case("mean", "nx/lib/nx.ex:9650-9654", lambda t: nx.mean(t), [([1, 2, 3], "s32")], [(2.0, "f32")], exact=False)
case("mean u8 axis 0", "nx/lib/nx.ex:9664-9668", lambda t: nx.mean(t, axes=[0]), [([1, 2, 3], "u8")], [(2.0, "f32")], exact=False)
case("mean axis 0 of iota {2,2,3}", "nx/lib/nx.ex:9670-9678", lambda t: nx.mean(t, axes=[0]), [(_I223, "s32")],
     [([[3.0, 4.0, 5.0], [6.0, 7.0, 8.0]], "f32")], exact=False)
case("mean axes 0,2", "nx/lib/nx.ex:9680-9685", lambda t: nx.mean(t, axes=[0, 2]), [(_I223, "s32")], [([4.0, 7.0], "f32")], exact=False)
case("mean axis -1", "nx/lib/nx.ex:9687-9695", lambda t: nx.mean(t, axes=[-1]), [(_I223, "s32")], [([[1.0, 4.0], [7.0, 10.0]], "f32")],
     exact=False)
case("mean axis -1 keep", "nx/lib/nx.ex:9699-9715", lambda t: nx.mean(t, axes=[-1], keep_axes=True), [(_I223, "s32")],
     [([[[1.0], [4.0]], [[7.0], [10.0]]], "f32")], exact=False)
case("logical_not s32", "nx/lib/nx.ex:7332-7336", lambda t: nx.logical_not(t), [([-1, 0, 1], "s32")], [([0, 1, 0], "u8")])
case("logical_not f32", "nx/lib/nx.ex:7338-7342", lambda t: nx.logical_not(t), [([-1.0, 0.0, 1.0], "f32")], [([0, 1, 0], "u8")])
case("not_equal", "nx/lib/nx.ex:7413-7419", lambda a, b: nx.not_equal(a, b), [([1, 1, 2], "s32"), ([1, 2, 3], "s32")], [([0, 1, 1], "u8")])
case("not_equal matrices", "nx/lib/nx.ex:7421-7430", lambda a, b: nx.not_equal(a, b),
     [([[1, 4, 2], [4, 5, 6]], "s32"), ([[1, 3, 2], [4, 2, 1]], "s32")], [([[0, 1, 0], [0, 1, 1]], "u8")])
_I52 = [[0, 1], [2, 3], [4, 5], [6, 7], [8, 9]]
_I25 = [[0, 1, 2, 3, 4], [5, 6, 7, 8, 9]]
case("slice_along_axis axis 0", "nx/lib/nx.ex:14324-14331", lambda t: nx.slice_along_axis(t, 1, 2, axis=0), [(_I52, "s32")],
     [([[2, 3], [4, 5]], "s32")])
case("slice_along_axis axis 1", "nx/lib/nx.ex:14333-14340", lambda t: nx.slice_along_axis(t, 1, 2, axis=1), [(_I25, "s32")],
     [([[1, 2], [6, 7]], "s32")])
case("slice_along_axis tensor start", "nx/lib/nx.ex:14350-14356", lambda t, s: nx.slice_along_axis(t, s, 1, axis=0), [(_I25, "s32"), (0, "s32")],
     [([[0, 1, 2, 3, 4]], "s32")])
case("slice_along_axis strides", "nx/lib/nx.ex:14358-14365", lambda t: nx.slice_along_axis(t, 0, 3, axis=-1, strides=2), [(_I25, "s32")],
     [([[0, 2], [5, 7]], "s32")])

# ---- binary broadcast: nx/test/nx_test.exs:37-147 (each pair in both orders, as the test's `commute` does) ----
_BROADCASTS = [
    ("{2,1} + {1,2}", "nx/test/nx_test.exs:38-47", [[1], [2]], [[10, 20]], [[11, 21], [12, 22]]),
    ("{2} + {2,2}", "nx/test/nx_test.exs:49-58", [1, 2], [[1, 2], [3, 4]], [[2, 4], [4, 6]]),
    ("{1,2,1} + {2,1,2}", "nx/test/nx_test.exs:60-74", [[[10], [20]]], [[[1, 2]], [[3, 4]]], [[[11, 12], [21, 22]], [[13, 14], [23, 24]]]),
    ("{1,3,1} + {4,1,3}", "nx/test/nx_test.exs:76-96", [[[100], [200], [300]]], [[[1, 2, 3]], [[4, 5, 6]], [[7, 8, 9]], [[10, 11, 12]]],
     [[[101, 102, 103], [201, 202, 203], [301, 302, 303]], [[104, 105, 106], [204, 205, 206], [304, 305, 306]],
      [[107, 108, 109], [207, 208, 209], [307, 308, 309]], [[110, 111, 112], [210, 211, 212], [310, 311, 312]]]),
    ("{1,2,2,1} + {2,1,2}", "nx/test/nx_test.exs:98-112", [[[[10], [20]], [[30], [40]]]], [[[1, 2]], [[3, 4]]],
     [[[[11, 12], [21, 22]], [[33, 34], [43, 44]]]]),
    ("{1,2,2,1} + {2,1,1,2}", "nx/test/nx_test.exs:114-130", [[[[10], [20]], [[30], [40]]]], [[[[1, 2]]], [[[3, 4]]]],
     [[[[11, 12], [21, 22]], [[31, 32], [41, 42]]], [[[13, 14], [23, 24]], [[33, 34], [43, 44]]]]),
    ("{2,2,1} + {2,1,2}", "nx/test/nx_test.exs:132-146", [[[10], [20]], [[30], [40]]], [[[1, 2]], [[3, 4]]],
     [[[11, 12], [21, 22]], [[33, 34], [43, 44]]]),
]
for _name, _cite, _a, _b, _want in _BROADCASTS:
    case("broadcast add " + _name, _cite, lambda a, b: nx.add(a, b), [(_a, "s32"), (_b, "s32")], [(_want, "s32")])
    case("broadcast add " + _name + " (commuted)", _cite, lambda a, b: nx.add(a, b), [(_b, "s32"), (_a, "s32")], [(_want, "s32")])

# ---- reduce_min / reduce_max over non-finite rows: nx/test/nx_test.exs:1645-1744 -------------------------
case("reduce_min non-finite", "nx/test/nx_test.exs:1646-1678", lambda t: nx.reduce_min(t, axes=[1]), [(NONFINITE, "f32")],
     [([-INF, NAN, -INF, -INF, 1, NAN, -INF, 0, NAN, NAN, NAN, NAN], "f32")])
case("reduce_max non-finite", "nx/test/nx_test.exs:1711-1743", lambda t: nx.reduce_max(t, axes=[1]), [(NONFINITE, "f32")],
     [([INF, NAN, 1, 1, INF, NAN, INF, INF, NAN, NAN, NAN, NAN], "f32")])
case("reduce_min all axes / axis 0 / keep", "nx/test/nx_test.exs:1680-1707",
     lambda t: (nx.reduce_min(t), nx.reduce_min(t, axes=[0]), nx.reduce_min(t, axes=[0], keep_axes=True), nx.reduce_min(t, keep_axes=True)),
     [([[1, 2, 3], [3, 1, 2]], "s32")], [(1, "s32"), ([1, 1, 2], "s32"), ([[1, 1, 2]], "s32"), ([[1]], "s32")])

# ---- dot with general contraction and batch axes: nx/test/nx_test.exs:1877-1975 -----------------------------
case("dot by a scalar", "nx/test/nx_test.exs:1878-1884", lambda t: nx.dot(t, 3), [([[1, 2, 3]], "s32")], [([[3, 6, 9]], "s32")])
case("dot/4 keeps the order of the contracting axes", "nx/test/nx_test.exs:1888-1910",
     lambda a, b: nx.dot(a, [3, 1, 2], [], b, [2, 3, 1], []),
     [(_iota_list((2, 7, 8, 3, 1)), "s32"), (_iota_list((1, 8, 3, 7, 3)), "s32")],
     [([[[[3731448, 3745476, 3759504]]], [[[10801560, 10843812, 10886064]]]], "s32")])
case("dot/6 batched, different free sizes", "nx/test/nx_test.exs:1914-1920",
     lambda a, b: nx.dot(a, [1, 2], [0], b, [2, 1], [0]),
     [(_iota_list((3, 2, 4, 1)), "s32"), (_iota_list((3, 4, 2, 2)), "s32")], [([[[252, 280]], [[2172, 2264]], [[6140, 6296]]], "s32")])
case("dot/6 two batch axes", "nx/test/nx_test.exs:1922-1966",
     lambda a, b: nx.dot(a, [2], [0, 1], b, [3], [0, 1]),
     [(_iota_list((3, 2, 1, 3, 2)), "s32"), (_iota_list((3, 2, 1, 1, 4)), "s32")],
     [([[[[[[0, 0, 0, 0]], [[0, 1, 2, 3]]], [[[0, 2, 4, 6]], [[0, 3, 6, 9]]], [[[0, 4, 8, 12]], [[0, 5, 10, 15]]]],
         [[[[24, 30, 36, 42]], [[28, 35, 42, 49]]], [[[32, 40, 48, 56]], [[36, 45, 54, 63]]], [[[40, 50, 60, 70]], [[44, 55, 66, 77]]]]],
        [[[[[96, 108, 120, 132]], [[104, 117, 130, 143]]], [[[112, 126, 140, 154]], [[120, 135, 150, 165]]],
          [[[128, 144, 160, 176]], [[136, 153, 170, 187]]]],
         [[[[216, 234, 252, 270]], [[228, 247, 266, 285]]], [[[240, 260, 280, 300]], [[252, 273, 294, 315]]],
          [[[264, 286, 308, 330]], [[276, 299, 322, 345]]]]],
        [[[[[384, 408, 432, 456]], [[400, 425, 450, 475]]], [[[416, 442, 468, 494]], [[432, 459, 486, 513]]],
          [[[448, 476, 504, 532]], [[464, 493, 522, 551]]]],
         [[[[600, 630, 660, 690]], [[620, 651, 682, 713]]], [[[640, 672, 704, 736]], [[660, 693, 726, 759]]],
          [[[680, 714, 748, 782]], [[700, 735, 770, 805]]]]]], "s32")])
case("dot/6 batch axis of size 1", "nx/test/nx_test.exs:1968-1971", lambda t: nx.dot(t, [2], [0], t, [2], [0]),
     [([[[1, 2, 3], [4, 5, 6]]], "s32")], [([[[14, 32], [32, 77]]], "s32")])

# ---- clip with infinite bounds, concatenate along a middle axis: nx/test/nx_test.exs:2308-2344 -------------
case("clip with infinite bounds", "nx/test/nx_test.exs:2308-2311", lambda t: nx.clip(t, -INF, INF), [([1.0, 2.0, 3.0], "f32")],
     [([1.0, 2.0, 3.0], "f32")])
case("concatenate middle axis", "nx/test/nx_test.exs:2317-2342",
     lambda t: nx.concatenate([t, nx.add(t, 10), nx.add(t, 20)], axis=1), [(_iota_list((2, 2, 2)), "s32")],
     [([[[0, 1], [2, 3], [10, 11], [12, 13], [20, 21], [22, 23]], [[4, 5], [6, 7], [14, 15], [16, 17], [24, 25], [26, 27]]], "s32")])

# ---- window aggregates with "same" padding, strides and dilations: nx/test/nx_test.exs:828-960 -------------
case("window_sum strides, padding, dilations", "nx/test/nx_test.exs:829-855",
     lambda t: nx.window_sum(t, (2, 1, 2), strides=[2, 1, 1], padding=[(2, 1), (3, 1), (1, 0)], window_dilations=[1, 2, 2]),
     [([[[4, 2, 1, 3], [4, 2, 1, 7]], [[1, 2, 5, 7], [1, 8, 9, 2]]], "s32")],
     [([[[0, 0, 0]] * 6, [[0, 0, 0], [0, 0, 0], [0, 0, 0], [4, 11, 14], [10, 15, 19], [0, 0, 0]]], "s32")])
_I33 = _iota_list((3, 3))
case("window_sum same f64", "nx/test/nx_test.exs:857-862", lambda t: nx.window_sum(t, (2, 1), padding="same"), [(_I33, "f64")],
     [([[3.0, 5.0, 7.0], [9.0, 11.0, 13.0], [6.0, 7.0, 8.0]], "f64")])
case("window_product same f64", "nx/test/nx_test.exs:864-869", lambda t: nx.window_product(t, (2, 1), padding="same"), [(_I33, "f64")],
     [([[0.0, 4.0, 10.0], [18.0, 28.0, 40.0], [6.0, 7.0, 8.0]], "f64")])
case("window_max same f64", "nx/test/nx_test.exs:871-876", lambda t: nx.window_max(t, (2, 1), padding="same"), [(_I33, "f64")],
     [([[3, 4, 5], [6, 7, 8], [6, 7, 8]], "f64")])
case("window_min same f64", "nx/test/nx_test.exs:941-946", lambda t: nx.window_min(t, (2, 1), padding="same"), [(_I33, "f64")],
     [([[0.0, 1.0, 2.0], [3.0, 4.0, 5.0], [6.0, 7.0, 8.0]], "f64")])
case("window_max same, large kernel, strides", "nx/test/nx_test.exs:878-888",
     lambda t: nx.window_max(t, (1, 3, 3, 1), padding="same", strides=[1, 2, 2, 1]), [(_iota_list((1, 4, 4, 1)), "f32")],
     [([[[[5.0], [7.0]], [[13.0], [15.0]]]], "f32")])
case("window_max same, asymmetric kernel", "nx/test/nx_test.exs:890-900",
     lambda t: nx.window_max(t, (1, 2, 3, 1), padding="same", strides=[1, 2, 2, 1]), [(_iota_list((1, 4, 6, 1)), "f32")],
     [([[[[7.0], [9.0], [11.0]], [[19.0], [21.0], [23.0]]]], "f32")])
case("window_max same, kernel larger than input", "nx/test/nx_test.exs:902-907",
     lambda t: nx.window_max(t, (1, 3, 3, 1), padding="same", strides=[1, 1, 1, 1]), [(_iota_list((1, 2, 2, 1)), "f32")],
     [([[[[3.0], [3.0]], [[3.0], [3.0]]]], "f32")])
case("window_max same, kernel equal to input", "nx/test/nx_test.exs:909-914",
     lambda t: nx.window_max(t, (4, 4), padding="same", strides=[2, 2]), [(_iota_list((4, 4)), "f32")], [([[10.0, 11.0], [14.0, 15.0]], "f32")])
case("window_max same 1D", "nx/test/nx_test.exs:916-921", lambda t: nx.window_max(t, (3,), padding="same", strides=[2]),
     [(_iota_list((8,)), "f32")], [([1.0, 3.0, 5.0, 7.0], "f32")])
case("window_max same 2D", "nx/test/nx_test.exs:923-928", lambda t: nx.window_max(t, (3, 3), padding="same", strides=[2, 2]),
     [(_iota_list((4, 4)), "f32")], [([[5.0, 7.0], [13.0, 15.0]], "f32")])
case("window_max same, stride larger than kernel", "nx/test/nx_test.exs:930-935",
     lambda t: nx.window_max(t, (1, 2, 2, 1), padding="same", strides=[1, 3, 3, 1]), [(_iota_list((1, 6, 6, 1)), "f32")],
     [([[[[7.0], [10.0]], [[25.0], [28.0]]]], "f32")])
case("window_min same, large kernel", "nx/test/nx_test.exs:937-942",
     lambda t: nx.window_min(t, (1, 3, 3, 1), padding="same", strides=[1, 2, 2, 1]), [(_iota_list((1, 4, 4, 1)), "f32")],
     [([[[[0.0], [1.0]], [[4.0], [5.0]]]], "f32")])
case("window_max dilations, strides, same", "nx/test/nx_test.exs:948-958",
     lambda t: nx.window_max(t, (1, 2, 2, 1), padding="same", strides=[1, 2, 2, 1], window_dilations=[1, 2, 2, 1]),
     [(_iota_list((1, 4, 4, 1)), "f32")], [([[[[5.0], [7.0]], [[13.0], [15.0]]]], "f32")])

# ---- sort / argsort along a leading axis: nx/test/nx_test.exs:2350-2466 ---------------------------------
_S432 = [[[4, 5], [2, 5], [5, 0]], [[1, 9], [2, 1], [2, 1]], [[0, -1], [-1, 0], [0, -1]], [[-1, 0], [0, -1], [-1, 0]]]
case("sort 1D", "nx/test/nx_test.exs:2351-2354", lambda t: nx.sort(t), [([3, 2, 1, 0], "s32")], [([0, 1, 2, 3], "s32")])
case("sort axis 0 of {4,3,2}", "nx/test/nx_test.exs:2356-2410", lambda t: nx.sort(t, axis=0), [(_S432, "s32")],
     [([[[-1, -1], [-1, -1], [-1, -1]], [[0, 0], [0, 0], [0, 0]], [[1, 5], [2, 1], [2, 0]], [[4, 9], [2, 5], [5, 1]]], "s32")])
case("argsort axis 0 of {4,3,2}", "nx/test/nx_test.exs:2428-2466", lambda t: nx.argsort(t, axis=0), [(_S432, "s32")],
     [([[[3, 2], [2, 3], [3, 2]], [[2, 3], [3, 2], [2, 0]], [[1, 0], [0, 1], [1, 3]], [[0, 1], [1, 0], [0, 1]]], "s32")])

# ---- convolution, valid padding: nx/test/nx_test.exs:155-258 ----------------------------------------------
_C2244 = _iota_list((2, 2, 4, 4))
case("conv valid, 2x2 kernel", "nx/test/nx_test.exs:156-180", lambda t, k: nx.conv(t, k, strides=[1, 1], padding="valid"),
     [(_C2244, "f32"), (_iota_list((1, 2, 2, 2)), "f32")],
     [([[[[440.0, 468.0, 496.0], [552.0, 580.0, 608.0], [664.0, 692.0, 720.0]]],
        [[[1336.0, 1364.0, 1392.0], [1448.0, 1476.0, 1504.0], [1560.0, 1588.0, 1616.0]]]], "f32")], exact=False)
case("conv valid, kernel as large as the input, 8 filters", "nx/test/nx_test.exs:182-207",
     lambda t, k: nx.conv(t, k, strides=[1, 1], padding="valid"), [(_C2244, "f32"), (_iota_list((8, 2, 4, 4)), "f32")],
     [([[[[10416.0]], [[26288.0]], [[42160.0]], [[58032.0]], [[73904.0]], [[89776.0]], [[105648.0]], [[121520.0]]],
        [[[26288.0]], [[74928.0]], [[123568.0]], [[172208.0]], [[220848.0]], [[269488.0]], [[318128.0]], [[366768.0]]]], "f32")], exact=False)
case("conv valid, 3x3 kernel, 2 filters", "nx/test/nx_test.exs:209-236", lambda t, k: nx.conv(t, k, strides=[1, 1], padding="valid"),
     [(_C2244, "f32"), (_iota_list((2, 2, 3, 3)), "f32")],
     [([[[[2793.0, 2946.0], [3405.0, 3558.0]], [[7005.0, 7482.0], [8913.0, 9390.0]]],
        [[[7689.0, 7842.0], [8301.0, 8454.0]], [[22269.0, 22746.0], [24177.0, 24654.0]]]], "f32")], exact=False)
case("conv valid, strides 2x1", "nx/test/nx_test.exs:239-258", lambda t, k: nx.conv(t, k, strides=[2, 1], padding="valid"),
     [(_C2244, "f32"), (_iota_list((1, 2, 2, 2)), "f32")],
     [([[[[440.0, 468.0, 496.0], [664.0, 692.0, 720.0]]], [[[1336.0, 1364.0, 1392.0], [1560.0, 1588.0, 1616.0]]]], "f32")], exact=False)

# ---- eye: exla/test/exla/defn/expr_test.exs:3260-3272, nx/lib/nx.ex:1278-1332 ------------------------------
case("eye 2", "exla/test/exla/defn/expr_test.exs:3261-3265", lambda t: nx.add(nx.eye(2), t), [(0, "s32")], [([[1, 0], [0, 1]], "s32")])
case("eye with type", "exla/test/exla/defn/expr_test.exs:3267-3271", lambda t: nx.add(nx.eye(1, type="f32"), t), [(0.0, "f32")], [([[1.0]], "f32")])
case("eye f32 3", "nx/lib/nx.ex:1287-1295", lambda t: nx.add(nx.eye(3, type="f32"), t), [(0.0, "f32")],
     [([[1.0, 0.0, 0.0], [0.0, 1.0, 0.0], [0.0, 0.0, 1.0]], "f32")])
case("eye {1,2}", "nx/lib/nx.ex:1299-1305", lambda t: nx.add(nx.eye((1, 2)), t), [(0, "s32")], [([[1, 0]], "s32")])
case("eye batched {2,4,3}", "nx/lib/nx.ex:1310-1327", lambda t: nx.add(nx.eye((2, 4, 3)), t), [(0, "s32")],
     [([[[1, 0, 0], [0, 1, 0], [0, 0, 1], [0, 0, 0]]] * 2, "s32")])
