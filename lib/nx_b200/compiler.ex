defmodule NxB200 do
  @moduledoc """
  `Nx.Defn.Compiler` for B200 GPUs over `libnxb200.so`.

      config :nx, default_backend: NxB200.Backend
      config :nx, :default_defn_options, compiler: NxB200

  Callback contract: `nx/lib/nx/defn/compiler.ex:29-101`; behaviour modelled on `EXLA.Defn`
  (`exla/lib/exla/defn.ex:15-72,151-191`): the traced expression is walked once per cache key,
  memoised by node id (`defn.ex:659-668`), and turned into the byte string
  `nxb200_program_build` consumes (layout in `include/nxb200.h`); every later call resolves the
  argument thunks to device buffers, runs the program and wraps the result buffers in the output
  templates.  Results are always fresh tensors on `NxB200.Backend` (`defn.ex:387-393`).

  `:cond` is lowered to every branch plus selects, `:block` to its default implementation.  A function
  that holds a `:while`, a hook or a `:runtime_call` is not one program: it is walked by
  `Nx.Defn.Evaluator` over tensors of this backend, one program per operation (the tested stand-in
  `nx_b200/defn.py` cuts the expression at those nodes and compiles the pieces whole; that is not
  ported).  Not lowered: custom reducers (`:reduce`, `:window_reduce`, `:fun`) and `:conv` (the
  stand-in's front-end lowers it to pad + slices + dot before the compiler sees it).  These, and
  anything else the device cannot run, raise `ArgumentError` naming the operation; no operation
  is computed on the host.

  Not compiled in this repository's build (no Elixir in the image).
  """
  @behaviour Nx.Defn.Compiler

  alias Nx.Defn.{Composite, Expr}
  alias Nx.Tensor, as: T
  alias NxB200.NIF

  @cache :nx_b200_programs

  ## public conveniences (EXLA.jit/2, EXLA.jit_apply/3: exla/lib/exla.ex)

  def jit(fun, opts \\ []), do: Nx.Defn.jit(fun, Keyword.put(opts, :compiler, __MODULE__))
  def jit_apply(fun, args, opts \\ []), do: Nx.Defn.jit_apply(fun, args, Keyword.put(opts, :compiler, __MODULE__))

  ## Nx.Defn.Compiler callbacks

  @impl true
  def __partitions_options__(opts) do
    for device <- 0..(NIF.device_count() - 1)//1, do: Keyword.put(opts, :device, device)
  end

  @impl true
  def __to_backend__(opts), do: {NxB200.Backend, [device: opts[:device] || 0]}

  @impl true
  def __jit__(key, vars, fun, args_list, opts), do: __compile__(key, vars, fun, opts).(args_list)

  @impl true
  def __compile__(key, vars, fun, opts) do
    device = opts[:device] || 0
    # the donation marks are part of the key: a donating call must not reuse the
    # non-donating executable (exla/lib/exla/defn.ex:337-353)
    args_key = for %T{} = v <- vars, do: {v.type, v.shape, v.names, v.vectorized_axes, v.donatable?}

    built =
      cached({key, args_key, Keyword.drop(opts, [:device])}, fn ->
        t0 = System.monotonic_time()
        expr = fun.(vars)
        t1 = System.monotonic_time()
        outputs = Composite.flatten_list([expr])

        if host_control?(outputs) do
          :host
        else
          program = NIF.program_build(serialize(outputs, vars))
          t2 = System.monotonic_time()

          :telemetry.execute(
            [:nx_b200, :compilation],
            %{eval_time: t1 - t0, compile_time: t2 - t1, total_time: t2 - t0},
            %{key: key}
          )

          {program, expr}
        end
      end)

    case built do
      :host -> host_runner(key, vars, fun, opts, device)
      {program, expr} -> program_runner(program, expr, device)
    end
  end

  defp program_runner(program, expr, device) do
    fn args_list ->
      for args <- args_list do
        buffers = for thunk <- args, do: on_device(thunk.(), device).data.ref
        refs = NIF.program_run(program, device, buffers)

        {result, []} =
          Composite.traverse(expr, refs, fn %T{} = template, [ref | rest] ->
            {%{Nx.to_template(template) | data: %NxB200.Backend{ref: ref, device: device}}, rest}
          end)

        result
      end
    end
  end

  # A function with a loop or a host call in it (`:while`, `:io_call`, `:runtime_call`) is not one
  # program.  It is walked by `Nx.Defn.Evaluator` over tensors of this backend: every operation is
  # still a program on the device (`NxB200.Backend` runs each callback through this compiler), and
  # the loop condition, the hooks and the callbacks run on the host between them.  (The tested
  # stand-in `nx_b200/defn.py` does better: it cuts the expression at those nodes and compiles the
  # pieces whole.)
  defp host_runner(key, vars, fun, opts, device) do
    evaluate = Nx.Defn.Evaluator.__compile__(key, vars, fun, Keyword.take(opts, [:hooks, :garbage_collect]))

    fn args_list ->
      for args <- args_list do
        [result] = evaluate.([for(thunk <- args, do: fn -> on_device(thunk.(), device) end)])
        Composite.traverse(result, &on_device(&1, device))
      end
    end
  end

  defp on_device(%T{data: %NxB200.Backend{device: device}} = t, device), do: t
  defp on_device(%T{data: %NxB200.Backend{}} = t, device), do: Nx.backend_copy(t, {NxB200.Backend, device: device})
  defp on_device(%T{data: %Nx.BinaryBackend{}} = t, device), do: Nx.backend_copy(t, {NxB200.Backend, device: device})

  defp on_device(%T{data: %other{}}, _device) do
    raise ArgumentError, "cannot run on NxB200 a tensor allocated on #{inspect(other)}"
  end

  @host_ops [:while, :io_call, :runtime_call]

  defp host_control?(outputs) do
    {found, _seen} = Enum.reduce(outputs, {false, %{}}, &scan/2)
    found
  end

  defp scan(_tensor, {true, seen}), do: {true, seen}

  defp scan(%T{data: %Expr{id: id, op: op}} = t, {false, seen}) do
    cond do
      is_map_key(seen, id) ->
        {false, seen}

      op in @host_ops ->
        {true, seen}

      true ->
        {_args, acc} = Nx.Defn.Tree.apply_args(t, {false, Map.put(seen, id, true)}, fn arg, acc -> {arg, scan(arg, acc)} end)
        acc
    end
  end

  defp scan(_other, acc), do: acc

  ## program cache: one build per key, concurrent callers of the same key wait for it
  ## (the role of EXLA.Defn.LockedCache, exla/lib/exla/defn/locked_cache.ex:35-59)

  defp cached(key, fun) do
    table = ensure_table()

    case :ets.lookup(table, key) do
      [{^key, value}] ->
        value

      [] ->
        :global.trans({{__MODULE__, key}, self()}, fn ->
          case :ets.lookup(table, key) do
            [{^key, value}] ->
              value

            [] ->
              value = fun.()
              :ets.insert(table, {key, value})
              value
          end
        end, [node()])
    end
  end

  defp ensure_table do
    case :ets.whereis(@cache) do
      :undefined ->
        try do
          :ets.new(@cache, [:named_table, :public, :set, read_concurrency: true])
        rescue
          ArgumentError -> @cache
        end

      _ ->
        @cache
    end
  end

  ## Expr -> program bytes

  @doc false
  def serialize(outputs, vars) do
    # parameters first, in argument order, so that the program keeps the function's arity
    # `scope` maps a parameter position to the node that carries its value: the program's own
    # parameters at the top, a block's arguments while its default implementation is lowered
    state = %{nodes: [], index: %{}, count: 0, scope: %{}}

    state =
      vars
      |> Composite.flatten_list()
      |> Enum.with_index()
      |> Enum.reduce(state, fn {%T{} = v, i}, st ->
        {node, st} = emit(st, {:parameter, i}, "parameter", v, [], [i], [], <<>>)
        %{st | scope: Map.put(st.scope, i, node)}
      end)

    {out_indices, state} = Enum.map_reduce(outputs, state, &visit/2)
    donated = donation_pairs(vars, outputs)

    [
      "NXB1",
      <<state.count::little-32>>,
      Enum.reverse(state.nodes),
      <<length(out_indices)::little-32>>,
      for(i <- out_indices, do: <<i::little-32>>),
      if(donated == [], do: [], else: [<<length(donated)::little-32>>, for({p, o} <- donated, do: <<p::little-32, o::little-32>>)])
    ]
  end

  # pairs each donated argument with the first unused output of its type and shape
  # (exla/lib/exla/defn.ex:598-645)
  defp donation_pairs(vars, outputs) do
    outs = Enum.with_index(outputs)

    {pairs, _used} =
      vars
      |> Composite.flatten_list()
      |> Enum.with_index()
      |> Enum.filter(fn {v, _} -> v.donatable? end)
      |> Enum.map_reduce(MapSet.new(), fn {v, p}, used ->
        case Enum.find(outs, fn {o, i} -> not MapSet.member?(used, i) and o.type == v.type and o.shape == v.shape end) do
          {_, i} ->
            {{p, i}, MapSet.put(used, i)}

          nil ->
            raise ArgumentError,
                  "a tensor of type #{inspect(v.type)} and shape #{inspect(v.shape)} was marked as donatable " <>
                    "but no output with the same type and shape is available to take over its buffer"
        end
      end)

    pairs
  end

  defp visit(%T{data: %Expr{id: id}} = t, state) do
    case state.index do
      %{^id => i} -> {i, state}
      %{} -> lower(Nx.devectorize(t), state)
    end
  end

  defp emit(state, id, op, %T{type: type, shape: shape}, args, ints, flts, blob) do
    dims = Tuple.to_list(shape)

    node = [
      <<byte_size(op)::8>>, op,
      <<NIF.type_code(type)::8, length(dims)::8>>, for(d <- dims, do: <<d::little-signed-64>>),
      <<length(args)::little-16>>, for(a <- args, do: <<a::little-32>>),
      <<length(ints)::little-16>>, for(i <- ints, do: <<i::little-signed-64>>),
      <<length(flts)::little-16>>, for(f <- flts, do: encode_float(f)),
      <<byte_size(blob)::little-64>>, blob
    ]

    i = state.count
    {i, %{state | nodes: [node | state.nodes], index: Map.put(state.index, id, i), count: i + 1}}
  end

  defp encode_float(:nan), do: <<0x7FF8000000000000::little-64>>
  defp encode_float(:infinity), do: <<0x7FF0000000000000::little-64>>
  defp encode_float(:neg_infinity), do: <<0xFFF0000000000000::little-64>>
  defp encode_float(f), do: <<f * 1.0::little-float-64>>

  defp args(tensors, state), do: Enum.map_reduce(tensors, state, &visit/2)

  # node `i` (the value of `tensor`) as `type`: itself, or an as_type node filed under `id`
  defp converted(state, _id, i, %T{type: type}, type), do: {i, state}
  defp converted(state, id, i, %T{} = tensor, type), do: emit(state, id, "as_type", %{tensor | type: type}, [i], [], [], <<>>)

  defp simple(%T{data: %Expr{id: id, op: op}} = t, tensors, ints, state) do
    {idx, state} = args(tensors, state)
    emit(state, id, Atom.to_string(op), t, idx, ints, [], <<>>)
  end

  @elementwise [:exp, :expm1, :log, :log1p, :sigmoid, :cos, :sin, :tan, :cosh, :sinh, :tanh, :acos, :asin, :atan,
                :acosh, :asinh, :atanh, :sqrt, :rsqrt, :cbrt, :erf, :erfc, :erf_inv, :abs, :bitwise_not, :ceil, :floor,
                :negate, :round, :sign, :count_leading_zeros, :population_count, :is_nan, :is_infinity, :as_type,
                :add, :subtract, :multiply, :divide, :pow, :remainder, :atan2, :min, :max, :quotient, :bitwise_and,
                :bitwise_or, :bitwise_xor, :left_shift, :right_shift, :equal, :not_equal, :greater, :less,
                :greater_equal, :less_equal, :logical_and, :logical_or, :logical_xor, :select, :clip, :reshape]

  defp lower(%T{data: %Expr{id: id, op: :parameter, args: [i]}}, state) do
    # written up front by serialize/2, or an argument of the block being lowered
    node = Map.fetch!(state.scope, i)
    {node, %{state | index: Map.put(state.index, id, node)}}
  end

  defp lower(%T{data: %Expr{id: id, op: :constant, args: [number]}, type: type} = t, state) do
    if Nx.Type.float?(type),
      do: emit(state, id, "constant", t, [], [], [number], <<>>),
      else: emit(state, id, "constant", t, [], [number], [], <<>>)
  end

  defp lower(%T{data: %Expr{id: id, op: :tensor, args: [literal]}} = t, state) do
    emit(state, id, "tensor", t, [], [], [], Nx.to_binary(literal))
  end

  defp lower(%T{data: %Expr{id: id, op: :metadata, args: [inner, _meta]}} = t, state) do
    {[i], state} = args([inner], state)
    emit(state, id, "metadata", t, [i], [], [], <<>>)
  end

  defp lower(%T{data: %Expr{op: op, args: tensors}} = t, state) when op in @elementwise do
    simple(t, tensors, [], state)
  end

  defp lower(%T{data: %Expr{op: op, args: [x, opts]}} = t, state)
       when op in [:sum, :product, :reduce_max, :reduce_min, :all, :any] do
    axes = opts[:axes] || Nx.axes(x)
    simple(t, [x], [bool(opts[:keep_axes]), length(axes) | axes], state)
  end

  defp lower(%T{data: %Expr{op: op, args: [x, opts]}} = t, state) when op in [:argmax, :argmin] do
    simple(t, [x], [bool(opts[:tie_break] == :high), opts[:axis] || -1, bool(opts[:keep_axis])], state)
  end

  defp lower(%T{data: %Expr{op: :dot, args: [a, c1, b1, b, c2, b2]}} = t, state) do
    simple(t, [a, b], Enum.flat_map([c1, b1, c2, b2], &[length(&1) | &1]), state)
  end

  defp lower(%T{data: %Expr{op: :squeeze, args: [x, axes]}} = t, state), do: simple(t, [x], [length(axes) | axes], state)
  defp lower(%T{data: %Expr{op: :broadcast, args: [x, _shape, axes]}} = t, state), do: simple(t, [x], [length(axes) | axes], state)
  defp lower(%T{data: %Expr{op: :transpose, args: [x, perm]}} = t, state), do: simple(t, [x], perm, state)
  defp lower(%T{data: %Expr{op: :reverse, args: [x, axes]}} = t, state), do: simple(t, [x], axes, state)
  defp lower(%T{data: %Expr{op: :iota, args: [axis]}} = t, state), do: simple(t, [], [axis || -1], state)

  # pieces are converted to the result's type first (exla/lib/exla/defn.ex, :concatenate and :stack)
  defp lower(%T{data: %Expr{id: id, op: :concatenate, args: [tensors, axis]}, type: type} = t, state) do
    {pieces, state} =
      tensors
      |> Enum.with_index()
      |> Enum.map_reduce(state, fn {piece, k}, st ->
        {i, st} = visit(piece, st)
        converted(st, {:piece, id, k}, i, piece, type)
      end)

    emit(state, id, "concatenate", t, pieces, [axis], [], <<>>)
  end

  # the device has no :stack: every piece gets a new axis of extent 1 (a reshape, which costs
  # nothing), then the pieces are concatenated along it
  defp lower(%T{data: %Expr{id: id, op: :stack, args: [tensors, axis]}, type: type} = t, state) do
    {pieces, state} =
      tensors
      |> Enum.with_index()
      |> Enum.map_reduce(state, fn {piece, k}, st ->
        {i, st} = visit(piece, st)
        {i, st} = converted(st, {:piece, id, k}, i, piece, type)
        shape = piece.shape |> Tuple.to_list() |> List.insert_at(axis, 1) |> List.to_tuple()
        emit(st, {:lifted, id, k}, "reshape", %{piece | type: type, shape: shape}, [i], [], [], <<>>)
      end)

    emit(state, id, "concatenate", t, pieces, [axis], [], <<>>)
  end

  defp lower(%T{data: %Expr{op: :slice, args: [x, starts, lengths, strides]}} = t, state) do
    if Enum.all?(starts, &is_integer/1) do
      simple(t, [x], starts ++ lengths ++ strides, state)
    else
      # dynamic starts: one scalar tensor per axis follows the operand, the attribute is ignored
      scalars = for s <- starts, do: if(is_integer(s), do: Expr.constant(Nx.template({}, {:s, 32}), s, []), else: s)
      simple(t, [x | scalars], List.duplicate(0, length(starts)) ++ lengths ++ strides, state)
    end
  end

  defp lower(%T{data: %Expr{op: :put_slice, args: [x, starts, slice]}} = t, state) do
    scalars = for s <- starts, do: if(is_integer(s), do: Expr.constant(Nx.template({}, {:s, 32}), s, []), else: s)
    simple(t, [x, slice | scalars], [], state)
  end

  defp lower(%T{data: %Expr{op: :pad, args: [x, value, config]}} = t, state) do
    {lo, hi, interior} = config |> Enum.map(&Tuple.to_list/1) |> Enum.zip() |> Enum.map(&Tuple.to_list/1) |> List.to_tuple()
    simple(t, [x, value], lo ++ hi ++ interior, state)
  end

  defp lower(%T{data: %Expr{op: :gather, args: [x, indices, opts]}} = t, state), do: simple(t, [x, indices], opts[:axes], state)

  # the device scatters into a copy of the target: target and updates arrive in the result's type,
  # the positions as s32 or s64 (the reference converts in its lowering too, exla/lib/exla/defn.ex:1829-1848)
  defp lower(%T{data: %Expr{id: id, op: op, args: [x, indices, updates, opts]}, type: type} = t, state)
       when op in [:indexed_add, :indexed_put] do
    {[xi, ii, ui], state} = args([x, indices, updates], state)
    {xi, state} = converted(state, {:target, id}, xi, x, type)
    {ui, state} = converted(state, {:updates, id}, ui, updates, type)
    index_type = if indices.type in [{:s, 64}, {:u, 64}], do: {:s, 64}, else: {:s, 32}
    {ii, state} = converted(state, {:positions, id}, ii, indices, index_type)
    emit(state, id, Atom.to_string(op), t, [xi, ii, ui], opts[:axes], [], <<>>)
  end

  defp lower(%T{data: %Expr{op: op, args: [x, window, opts]}} = t, state)
       when op in [:window_sum, :window_max, :window_min, :window_product] do
    rank = tuple_size(window)
    {lo, hi} = opts[:padding] |> Enum.unzip()
    dil = List.wrap(opts[:window_dilations] || List.duplicate(1, rank))
    simple(t, [x], Tuple.to_list(window) ++ opts[:strides] ++ lo ++ hi ++ dil, state)
  end

  defp lower(%T{data: %Expr{op: :sort, args: [x, opts]}} = t, state) do
    last_axis!(x, opts[:axis])
    simple(t, [x], [bool(opts[:direction] == :desc)], state)
  end

  defp lower(%T{data: %Expr{op: :argsort, args: [x, opts]}} = t, state) do
    last_axis!(x, opts[:axis])
    simple(t, [x], [bool(opts[:direction] == :desc), bool(opts[:stable])], state)
  end

  # ones where the last two coordinates agree: two iotas compared, as the reference lowers it
  # (exla/lib/exla/defn.ex:1120)
  defp lower(%T{data: %Expr{id: id, op: :eye, args: []}, shape: shape} = t, state) do
    rank = tuple_size(shape)
    index = %{t | type: {:s, 32}}
    {rows, state} = emit(state, {:eye_rows, id}, "iota", index, [], [rank - 2], [], <<>>)
    {cols, state} = emit(state, {:eye_cols, id}, "iota", index, [], [rank - 1], [], <<>>)
    {same, state} = emit(state, {:eye_same, id}, "equal", %{t | type: {:u, 8}}, [rows, cols], [], [], <<>>)
    emit(state, id, "as_type", t, [same], [], [], <<>>)
  end

  # :block (take, take_along_axis, top_k, logical_not, all_close, cumulative operations, …: nx/lib/nx.ex
  # `block/4`; nx/lib/nx/defn/expr.ex:826-842): the default implementation is lowered in place, its
  # parameters standing for the block's tensor arguments (the reference compiles it as a sub-computation
  # called with those arguments, exla/lib/exla/defn.ex:1055-1086).  An operation inside it that the
  # device lacks raises from its own node.
  defp lower(%T{data: %Expr{id: id, op: :block, args: [_struct, in_args, expr, _fun]}}, state) when not is_tuple(expr) do
    {node, state} = in_block_scope(in_args, state, &visit(expr, &1))
    {node, %{state | index: Map.put(state.index, id, node)}}
  end

  defp lower(%T{data: %Expr{id: id, op: :elem, args: [%T{data: %Expr{op: :block, args: [_struct, in_args, exprs, _fun]}}, i]}}, state) do
    {node, state} = in_block_scope(in_args, state, &visit(elem(exprs, i), &1))
    {node, %{state | index: Map.put(state.index, id, node)}}
  end

  # :cond inside one program: every branch is computed and the first clause whose predicate holds is
  # selected (what `defn.cond` of the tested stand-in does inside a traced function).  A branch that
  # holds a loop or a host call raises from that node.
  defp lower(%T{data: %Expr{id: id, op: :cond, args: [clauses, last]}} = t, state) when not is_tuple(last) do
    select_chain(id, t, clauses, last, state)
  end

  defp lower(%T{data: %Expr{id: id, op: :elem, args: [%T{data: %Expr{op: :cond, args: [clauses, last]}}, i]}} = t, state) do
    clauses = for {pred, body} <- clauses, do: {pred, elem(body, i)}
    select_chain(id, t, clauses, elem(last, i), state)
  end

  defp lower(%T{data: %Expr{op: :elem, args: [tuple, i]}}, state) do
    # multi-output nodes do not exist on the device: project at trace level
    visit(elem(tuple_of(tuple), i), state)
  end

  defp lower(%T{data: %Expr{op: op}}, _state) do
    raise ArgumentError,
          "NxB200 cannot compile the operation :#{op} (there is no CPU fallback; run it on another backend " <>
            "or outside of the compiled function)"
  end

  # runs `fun` with the block's tensor arguments (the leading elements of `in_args`; option lists
  # follow them) as parameters 0, 1, …, then restores the enclosing scope
  defp in_block_scope(in_args, state, fun) do
    {tensors, _opts} = Enum.split_while(in_args, &(not is_list(&1)))
    {nodes, state} = args(tensors, state)
    outer = state.scope
    inner = nodes |> Enum.with_index() |> Map.new(fn {node, pos} -> {pos, node} end)
    {result, state} = fun.(%{state | scope: inner})
    {result, %{state | scope: outer}}
  end

  # select(pred_1, body_1, select(pred_2, body_2, … last)), built from the last clause up; the
  # scalar predicates are broadcast to the result's shape first
  defp select_chain(id, %T{shape: shape} = t, clauses, last, state) do
    {acc, state} = visit(last, state)
    n = length(clauses)

    clauses
    |> Enum.reverse()
    |> Enum.with_index(1)
    |> Enum.reduce({acc, state}, fn {{pred, body}, k}, {acc, st} ->
      {p, st} = visit(pred, st)

      {p, st} =
        if shape == {},
          do: {p, st},
          else: emit(st, {:cond_pred, id, k}, "broadcast", %{pred | shape: shape}, [p], [0], [], <<>>)

      {b, st} = visit(body, st)
      emit(st, if(k == n, do: id, else: {:cond_step, id, k}), "select", t, [p, b, acc], [], [], <<>>)
    end)
  end

  defp tuple_of(%T{data: %Expr{op: :metadata, args: [inner, _]}}), do: tuple_of(inner)
  defp tuple_of(tuple) when is_tuple(tuple), do: tuple
  defp tuple_of(%T{data: %Expr{op: op}}), do: raise(ArgumentError, "NxB200 cannot compile the operation :#{op}")

  defp last_axis!(x, axis) do
    unless axis == Nx.rank(x) - 1 do
      raise ArgumentError, "NxB200 sorts along the last axis only; transpose the tensor first (got axis #{axis})"
    end
  end

  defp bool(true), do: 1
  defp bool(_), do: 0
end
