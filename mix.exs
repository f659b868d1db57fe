# Mix project of the Elixir side (backend + compiler modules over the NIF shim).
# NOT BUILT IN THIS REPOSITORY'S CI: the build image has no Erlang/OTP or Elixir.
# `mix compile` on a machine that has them builds c_src/nxb200_nif.c against
# include/nxb200.h and links nx_b200/libnxb200.so (see the make task below).
defmodule NxB200.MixProject do
  use Mix.Project

  def project do
    [
      app: :nx_b200,
      version: "0.1.0",
      elixir: "~> 1.17",
      compilers: [:nxb200_nif] ++ Mix.compilers(),
      deps: [{:nx, "~> 0.10"}]
    ]
  end

  def application, do: [extra_applications: [:logger]]
end

defmodule Mix.Tasks.Compile.Nxb200Nif do
  use Mix.Task.Compiler

  @impl true
  def run(_args) do
    erl_include = Path.join([:code.root_dir(), "usr", "include"])
    File.mkdir_p!("priv")

    args =
      ~w(-O2 -fPIC -shared -I#{erl_include} -Iinclude c_src/nxb200_nif.c -Lnx_b200 -l:libnxb200.so) ++
        ["-Wl,-rpath,$ORIGIN", "-o", "priv/libnxb200_nif.so"]

    case System.cmd("cc", args, stderr_to_stdout: true) do
      {_, 0} -> File.cp!("nx_b200/libnxb200.so", "priv/libnxb200.so"); {:ok, []}
      {out, _} -> Mix.raise("building the NIF shim failed:\n" <> out)
    end
  end
end
