defmodule NxB200.Backend do
  @moduledoc """
  `Nx.Backend` whose tensors live in B200 device memory behind `libnxb200.so`.

  Storage callbacks map one to one onto the buffer entry points of `include/nxb200.h`
  (the role `EXLA.DeviceBuffer` plays in `exla/lib/exla/backend.ex:43-83,222-226`).  Every
  compute callback is the compiler applied to a one-node expression, exactly as
  `EXLA.Backend` does it (`exla/lib/exla/backend.ex:363-431`): the callback builds the
  `Nx.Defn.Expr` node for the operation and runs it through `NxB200.jit_apply/3`.  A callback
  the compiler cannot lower raises; there is no host implementation to fall back to.

  Written to the callback arities of `nx/lib/nx/backend.ex:46-144`.  Not compiled in this
  repository's build (no Elixir in the image); `nx_b200/backend.py` is the tested stand-in.
  """
  @behaviour Nx.Backend
  @enforce_keys [:ref, :device]
  defstruct [:ref, :device]

  alias Nx.Tensor, as: T
  alias NxB200.Backend, as: B
  alias NxB200.NIF

  @impl true
  def init(opts), do: Keyword.validate!(opts, device: 0)

  ## storage

  @impl true
  def from_binary(%T{type: type, shape: shape} = out, binary, opts) do
    device = opts[:device] || 0
    ref = NIF.from_binary(device, NIF.type_code(type), shape, IO.iodata_to_binary(binary))
    put_in(out.data, %B{ref: ref, device: device})
  end

  @impl true
  def to_binary(%T{data: %B{ref: ref}, type: {_, bits}}, limit) do
    NIF.to_binary(ref, limit * div(max(bits, 8), 8))
  end

  @impl true
  def constant(out, number, opts) do
    Nx.BinaryBackend.constant(out, number, []) |> Nx.BinaryBackend.backend_transfer(__MODULE__, opts)
  end

  @impl true
  def backend_copy(%T{data: %B{ref: ref, device: from}} = t, __MODULE__, opts) do
    device = opts[:device] || 0

    if device == from do
      # a copy on the same device goes through the host, as the reference's does (backend.ex:54-56)
      from_binary(t, NIF.to_binary(ref, byte_size_of(t)), opts)
    else
      put_in(t.data, %B{ref: NIF.copy_to_device(ref, device), device: device})
    end
  end

  def backend_copy(%T{data: %B{ref: ref}} = t, backend, opts) do
    backend.from_binary(t, NIF.to_binary(ref, byte_size_of(t)), opts)
  end

  @impl true
  def backend_transfer(%T{data: %B{ref: ref, device: from}} = t, backend, opts) do
    if backend == __MODULE__ and (opts[:device] || 0) == from do
      t
    else
      try do
        backend_copy(t, backend, opts)
      after
        NIF.deallocate(ref)
      end
    end
  end

  @impl true
  def backend_deallocate(%T{data: %B{ref: ref}}) do
    case NIF.deallocate(ref) do
      :ok -> :ok
      {:error, :already_deallocated} -> :already_deallocated
    end
  end

  @impl true
  def to_pointer(%T{data: %B{ref: ref}} = t, opts \\ []) do
    opts = Keyword.validate!(opts, mode: :local, permissions: 0o400)

    case opts[:mode] do
      :local -> %Nx.Pointer{kind: :local, address: NIF.device_pointer(ref), data_size: byte_size_of(t)}
      :ipc -> %Nx.Pointer{kind: :ipc, handle: NIF.ipc_export(ref), data_size: byte_size_of(t)}
      other -> raise ArgumentError, "expected one of :local, :ipc, got: #{inspect(other)}"
    end
  end

  @impl true
  def from_pointer(%Nx.Pointer{} = pointer, type, shape, backend_opts, opts) do
    backend_opts = Keyword.validate!(backend_opts, device: 0)
    opts = Keyword.validate!(opts, [:names])
    template = Nx.template(shape, type, names: opts[:names])
    device = backend_opts[:device]

    if pointer.data_size != byte_size_of(template) do
      raise ArgumentError,
            "invalid pointer data_size for shape, expected #{byte_size_of(template)}, got: #{pointer.data_size}"
    end

    ref =
      case pointer do
        %Nx.Pointer{kind: :local, address: address} -> NIF.from_pointer(device, NIF.type_code(type), shape, address)
        %Nx.Pointer{kind: :ipc, handle: handle} -> NIF.from_ipc(device, NIF.type_code(type), shape, handle)
      end

    put_in(template.data, %B{ref: ref, device: device})
  end

  @impl true
  def to_batched(out, tensor, opts) do
    # slices are taken by the compiler; the last batch wraps around for leftover: :repeat
    leftover = opts[:leftover]
    batch_size = elem(out.shape, 0)
    axis_size = elem(tensor.shape, 0)
    remainder = rem(axis_size, batch_size)
    full = div(axis_size, batch_size)
    range = if remainder != 0 and leftover == :repeat, do: 0..full, else: 0..(full - 1)//1

    for i <- range do
      start = i * batch_size

      if start + batch_size <= axis_size do
        Nx.slice_along_axis(tensor, start, batch_size, axis: 0)
      else
        head = Nx.slice_along_axis(tensor, start, axis_size - start, axis: 0)
        tail = Nx.slice_along_axis(tensor, 0, batch_size - (axis_size - start), axis: 0)
        Nx.concatenate([head, tail], axis: 0)
      end
    end
  end

  @impl true
  def inspect(%T{data: %B{ref: ref}} = t, inspect_opts) do
    if NIF.is_deallocated(ref) do
      Inspect.Algebra.string(if t.donatable?, do: "Deallocated due to buffer donation", else: "Deallocated")
    else
      limit = if inspect_opts.limit == :infinity, do: :infinity, else: inspect_opts.limit + 1
      count = if limit == :infinity, do: Nx.size(t), else: min(limit, Nx.size(t))

      t
      |> to_binary(count)
      |> then(&Nx.Backend.inspect(t, &1, inspect_opts))
    end
  end

  defp byte_size_of(%T{type: {_, bits}} = t), do: Nx.size(t) * div(max(bits, 8), 8)

  ## compute: every callback is the compiler on a one-node expression (exla/lib/exla/backend.ex:363-431)

  binary_ops =
    [:add, :subtract, :multiply, :pow, :remainder, :divide, :atan2, :min, :max, :quotient] ++
      [:bitwise_and, :bitwise_or, :bitwise_xor, :left_shift, :right_shift] ++
      [:equal, :not_equal, :greater, :less, :greater_equal, :less_equal] ++
      [:logical_and, :logical_or, :logical_xor]

  unary_ops =
    [:exp, :expm1, :log, :log1p, :sigmoid, :cos, :sin, :tan] ++
      [:cosh, :sinh, :tanh, :acos, :asin, :atan, :acosh, :asinh, :atanh] ++
      [:sqrt, :rsqrt, :cbrt, :is_nan, :is_infinity, :erf, :erfc, :erf_inv] ++
      [:abs, :bitwise_not, :ceil, :conjugate, :floor, :negate, :round, :sign] ++
      [:count_leading_zeros, :population_count, :real, :imag]

  # {callback, arguments after `out`, which of them are tensors}
  callbacks =
    [
      {:eye, [:backend_options], []},
      {:iota, [:axis, :backend_options], []},
      {:as_type, [:tensor], [:tensor]},
      {:bitcast, [:tensor], [:tensor]},
      {:reshape, [:tensor], [:tensor]},
      {:squeeze, [:tensor, :axes], [:tensor]},
      {:broadcast, [:tensor, :shape, :axes], [:tensor]},
      {:transpose, [:tensor, :axes], [:tensor]},
      {:pad, [:tensor, :pad_value, :padding_config], [:tensor, :pad_value]},
      {:reverse, [:tensor, :axes], [:tensor]},
      {:dot, [:left, :c1, :b1, :right, :c2, :b2], [:left, :right]},
      {:clip, [:tensor, :min, :max], [:tensor, :min, :max]},
      {:gather, [:input, :indices, :opts], [:input, :indices]},
      {:select, [:pred, :on_true, :on_false], [:pred, :on_true, :on_false]},
      {:conv, [:tensor, :kernel, :opts], [:tensor, :kernel]},
      {:all, [:tensor, :opts], [:tensor]},
      {:any, [:tensor, :opts], [:tensor]},
      {:sum, [:tensor, :opts], [:tensor]},
      {:product, [:tensor, :opts], [:tensor]},
      {:reduce_max, [:tensor, :opts], [:tensor]},
      {:reduce_min, [:tensor, :opts], [:tensor]},
      {:argmax, [:tensor, :opts], [:tensor]},
      {:argmin, [:tensor, :opts], [:tensor]},
      {:reduce, [:tensor, :acc, :opts, :fun], [:tensor, :acc]},
      {:window_reduce, [:tensor, :acc, :shape, :opts, :fun], [:tensor, :acc]},
      {:window_sum, [:tensor, :shape, :opts], [:tensor]},
      {:window_product, [:tensor, :shape, :opts], [:tensor]},
      {:window_max, [:tensor, :shape, :opts], [:tensor]},
      {:window_min, [:tensor, :shape, :opts], [:tensor]},
      {:sort, [:tensor, :opts], [:tensor]},
      {:argsort, [:tensor, :opts], [:tensor]},
      {:window_scatter_max, [:tensor, :source, :init_value, :window_dims, :opts], [:tensor, :source, :init_value]},
      {:window_scatter_min, [:tensor, :source, :init_value, :window_dims, :opts], [:tensor, :source, :init_value]},
      {:indexed_add, [:tensor, :indices, :updates, :opts], [:tensor, :indices, :updates]},
      {:indexed_put, [:tensor, :indices, :updates, :opts], [:tensor, :indices, :updates]},
      {:triangular_solve, [:a, :b, :opts], [:a, :b]},
      {:fft, [:tensor, :opts], [:tensor]},
      {:ifft, [:tensor, :opts], [:tensor]}
    ] ++
      for(op <- binary_ops, do: {op, [:left, :right], [:left, :right]}) ++
      for(op <- unary_ops, do: {op, [:tensor], [:tensor]})

  for {name, args, tensor_args} <- callbacks do
    args = Enum.map(args, &Macro.var(&1, __MODULE__))
    tensor_args = Enum.map(tensor_args, &Macro.var(&1, __MODULE__))
    backend_options = Enum.find(args, [], &match?({:backend_options, _, _}, &1))

    @impl true
    def unquote(name)(out, unquote_splicing(args)) do
      out = Nx.to_template(out)

      expr_fun = fn unquote_splicing(tensor_args) ->
        Nx.Defn.Expr.unquote(name)(out, unquote_splicing(args))
      end

      jit(unquote(backend_options), expr_fun, [unquote_splicing(tensor_args)])
    end
  end

  @impl true
  def concatenate(out, tensors, axis) do
    out = Nx.to_template(out)
    jit([], fn tensors -> Nx.Defn.Expr.concatenate(out, Tuple.to_list(tensors), axis) end, [List.to_tuple(tensors)], tensors)
  end

  @impl true
  def stack(out, tensors, axis) do
    out = Nx.to_template(out)
    jit([], fn tensors -> Nx.Defn.Expr.stack(out, Tuple.to_list(tensors), axis) end, [List.to_tuple(tensors)], tensors)
  end

  @impl true
  def slice(out, tensor, start_indices, lengths, strides) do
    out = Nx.to_template(out)
    # dynamic start indices are tensor arguments of the one-node program
    dynamic = Enum.filter(start_indices, &is_struct(&1, T))

    jit(
      [],
      fn tensor, dynamic ->
        starts = fill_dynamic(start_indices, Tuple.to_list(dynamic))
        Nx.Defn.Expr.slice(out, tensor, starts, lengths, strides)
      end,
      [tensor, List.to_tuple(dynamic)],
      [tensor | dynamic]
    )
  end

  @impl true
  def put_slice(out, tensor, start_indices, slice) do
    out = Nx.to_template(out)
    dynamic = Enum.filter(start_indices, &is_struct(&1, T))

    jit(
      [],
      fn tensor, slice, dynamic ->
        Nx.Defn.Expr.put_slice(out, tensor, fill_dynamic(start_indices, Tuple.to_list(dynamic)), slice)
      end,
      [tensor, slice, List.to_tuple(dynamic)],
      [tensor, slice | dynamic]
    )
  end

  @impl true
  def block(struct, _output, args, fun) do
    # blocks run through their default implementation, which is made of the callbacks above
    apply(fun, [struct | args])
  end

  defp fill_dynamic(indices, dynamic) do
    {out, []} =
      Enum.map_reduce(indices, dynamic, fn
        %T{}, [d | rest] -> {d, rest}
        i, rest -> {i, rest}
      end)

    out
  end

  defp jit(opts, fun, args), do: jit(opts, fun, args, args)

  defp jit(opts, fun, args, tensors) do
    NxB200.jit_apply(fun, args, [on_conflict: :force] ++ device_opts(tensors, opts))
  end

  # the device of the first operand that already lives on one; mixing devices raises in the compiler
  defp device_opts(tensors, opts) do
    case for(%T{data: %B{device: d}} <- List.flatten(tensors), do: d) do
      [d | _] -> [device: d]
      [] -> [device: opts[:device] || 0]
    end
  end
end
