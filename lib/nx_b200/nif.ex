defmodule NxB200.NIF do
  @moduledoc """
  Stubs of the NIF shim `c_src/nxb200_nif.c` (one per entry point of `include/nxb200.h`).

  Mirrors the loading convention of the reference (`exla/lib/exla/nif.ex:5-21`): the shared
  object is loaded from `priv/` when the module is loaded, and every stub raises `:undef`
  until then (`nif.ex:108`).

  Not compiled in this repository's build (no Erlang/OTP in the image); the Python module
  `nx_b200/nif.py` binds the same C functions and is what the tests run.
  """
  @on_load :__on_load__

  def __on_load__ do
    path = :filename.join(:code.priv_dir(:nx_b200), ~c"libnxb200_nif")
    :erlang.load_nif(path, 0)
  end

  # devices
  def device_count, do: err()
  def device_synchronize(_device), do: err()

  # buffers: typespecs cross as {type_code, shape_tuple}
  def from_binary(_device, _type_code, _shape, _binary), do: err()
  def to_binary(_buffer, _byte_limit), do: err()
  def deallocate(_buffer), do: err()
  def is_deallocated(_buffer), do: err()
  def copy_to_device(_buffer, _device), do: err()
  def buffer_info(_buffer), do: err()
  def device_pointer(_buffer), do: err()
  def from_pointer(_device, _type_code, _shape, _address), do: err()
  def ipc_export(_buffer), do: err()
  def from_ipc(_device, _type_code, _shape, _handle), do: err()
  def buffer_alloc(_device, _type_code, _shape), do: err()
  # queued upload: `{:nxb200_upload_done, ref}` arrives at `pid` when the binary has been read
  def from_binary_async(_device, _type_code, _shape, _binary, _pid, _ref), do: err()
  # transfers that complete at the next device_synchronize, through a host region of the shim
  def host_region(_bytes), do: err()
  def region_write(_region, _binary), do: err()
  def region_binary(_region), do: err()
  def write_async(_buffer, _region, _bytes), do: err()
  def read_async(_buffer, _region, _bytes), do: err()

  # programs
  def program_build(_iodata), do: err()
  def program_outputs(_program), do: err()
  def program_run(_program, _device, _buffers), do: err()
  def program_describe(_program), do: err()
  def program_build_times(_program), do: err()
  def program_run_into(_program, _device, _arguments, _results), do: err()
  def program_kernel_source(_program, _index), do: err()
  def program_launch_count(_program), do: err()
  def dot_bf16_static_scratch(_device, _a, _b, _c, _m, _n, _k), do: err()

  # device timing, stream, self-test
  def timer_begin(_device), do: err()
  def timer_end(_device), do: err()
  def device_stream(_device), do: err()
  def selftest_bounded_wait(_device, _limit_us), do: err()

  # memory counters
  def memory_stats(_device), do: err()
  def memory_reset_peak(_device), do: err()

  # sharded execution
  def comm_id, do: err()
  def comm_init(_device, _rank, _world, _id), do: err()
  def comm_peer_alloc(_device, _elems), do: err()
  def comm_peer_open(_blobs), do: err()
  def comm_all_reduce_sum(_buffer), do: err()
  def comm_fused_launches, do: err()
  def comm_destroy, do: err()

  defp err, do: :erlang.nif_error(:undef)

  @type_codes %{
    {:u, 8} => 0, {:u, 16} => 1, {:u, 32} => 2, {:u, 64} => 3,
    {:s, 8} => 4, {:s, 16} => 5, {:s, 32} => 6, {:s, 64} => 7,
    {:f, 16} => 8, {:bf, 16} => 9, {:f, 32} => 10, {:f, 64} => 11
  }
  @code_types Map.new(@type_codes, fn {k, v} -> {v, k} end)

  @doc "`{kind, bits}` -> the `nxb200_dtype` code; raises for types the device does not hold."
  def type_code(type) do
    case @type_codes do
      %{^type => code} -> code
      _ -> raise ArgumentError, "NxB200 does not support tensors of type #{inspect(type)}"
    end
  end

  def code_type(code), do: Map.fetch!(@code_types, code)
end
