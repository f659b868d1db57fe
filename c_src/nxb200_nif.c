/*
 * Erlang NIF shim over libnxb200.so: one NIF per entry point of include/nxb200.h.
 *
 * NOT COMPILED IN THIS REPOSITORY'S BUILD: the image that builds and tests the library has no
 * Erlang/OTP (no erl_nif.h).  The file is written to the NIF API as documented and to the layout of
 * the reference's own shim; the Python module nx_b200/nif.py binds the same C entry points through
 * ctypes and is what the test-suite drives.
 *
 * Conventions taken from the reference (exla/c_src/exla/exla.cc, exla_nif_util.h):
 *   - handles are NIF resources; the resource destructor releases the native object when the BEAM
 *     collects the term (exla_client.cc:22-26);
 *   - an explicit deallocate marks the object deleted; a second one answers
 *     {:error, :already_deallocated} (exla.cc:462-475); any other use of a deleted buffer raises;
 *   - failures raise an Erlang exception carrying the native message (exla.cc:280-292):
 *     invalid arguments as ArgumentError, everything else as RuntimeError;
 *   - calls that touch the device or copy memory are dirty IO jobs, compilation is a dirty CPU job
 *     (exla.cc:323,445,453,475,524,624,634);
 *   - a typespec crosses as {type_code, shape_tuple}; type codes are the nxb200_dtype values.
 *
 * Build (on a machine with OTP):
 *   cc -O2 -fPIC -shared -I$ERL_ROOT/usr/include -Iinclude c_src/nxb200_nif.c \
 *      -Lnx_b200 -l:libnxb200.so -Wl,-rpath,'$ORIGIN' -o priv/libnxb200_nif.so
 */
#include <erl_nif.h>
#include <stdint.h>
#include <string.h>

#include "nxb200.h"

static ErlNifResourceType *BUF_TYPE, *PROG_TYPE;
static ERL_NIF_TERM atom_ok, atom_error, atom_already_deallocated, atom_true, atom_false;

typedef struct { nxb200_buffer *h; } buf_res;
typedef struct { nxb200_program *h; } prog_res;

static void buf_dtor(ErlNifEnv *env, void *p) { (void)env; buf_res *r = p; if (r->h) nxb200_buffer_release(r->h); }
static void prog_dtor(ErlNifEnv *env, void *p) { (void)env; prog_res *r = p; if (r->h) nxb200_program_release(r->h); }

/* ---- error mapping (exla.cc:280-292) ------------------------------------------------------ */

static ERL_NIF_TERM make_exception(ErlNifEnv *env, const char *module, const char *msg) {
  /* %Module{__exception__: true, message: msg} */
  ERL_NIF_TERM keys[3] = {enif_make_atom(env, "__struct__"), enif_make_atom(env, "__exception__"), enif_make_atom(env, "message")};
  ErlNifBinary b;
  size_t n = strlen(msg);
  enif_alloc_binary(n, &b);
  memcpy(b.data, msg, n);
  ERL_NIF_TERM vals[3] = {enif_make_atom(env, module), atom_true, enif_make_binary(env, &b)};
  ERL_NIF_TERM map;
  enif_make_map_from_arrays(env, keys, vals, 3, &map);
  return map;
}

static ERL_NIF_TERM raise_status(ErlNifEnv *env, int st) {
  char msg[4096];
  nxb200_last_error(msg, sizeof msg);
  if (st == NXB_ERR_ALREADY_DEALLOCATED) return enif_make_tuple2(env, atom_error, atom_already_deallocated);
  const char *module = (st == NXB_ERR_INVALID_ARGUMENT || st == NXB_ERR_UNSUPPORTED) ? "Elixir.ArgumentError" : "Elixir.RuntimeError";
  return enif_raise_exception(env, make_exception(env, module, msg));
}

/* ---- argument decoding ------------------------------------------------------------------------ */

static int get_shape(ErlNifEnv *env, ERL_NIF_TERM t, int64_t *dims, int *rank) {
  const ERL_NIF_TERM *e;
  int n;
  if (!enif_get_tuple(env, t, &n, &e) || n > NXB_MAX_RANK) return 0;
  for (int i = 0; i < n; ++i) {
    ErlNifSInt64 v;
    if (!enif_get_int64(env, e[i], &v)) return 0;
    dims[i] = v;
  }
  *rank = n;
  return 1;
}

static ERL_NIF_TERM make_shape(ErlNifEnv *env, const int64_t *dims, int rank) {
  ERL_NIF_TERM e[NXB_MAX_RANK];
  for (int i = 0; i < rank; ++i) e[i] = enif_make_int64(env, dims[i]);
  return enif_make_tuple_from_array(env, e, rank);
}

static nxb200_buffer *get_buf(ErlNifEnv *env, ERL_NIF_TERM t) {
  buf_res *r;
  return enif_get_resource(env, t, BUF_TYPE, (void **)&r) ? r->h : NULL;
}

static nxb200_program *get_prog(ErlNifEnv *env, ERL_NIF_TERM t) {
  prog_res *r;
  return enif_get_resource(env, t, PROG_TYPE, (void **)&r) ? r->h : NULL;
}

static ERL_NIF_TERM wrap_buf(ErlNifEnv *env, nxb200_buffer *b) {
  buf_res *r = enif_alloc_resource(BUF_TYPE, sizeof *r);
  r->h = b;
  ERL_NIF_TERM t = enif_make_resource(env, r);
  enif_release_resource(r);
  return t;
}

#define BADARG(env) enif_make_badarg(env)

/* ---- devices -------------------------------------------------------------------------------------- */

/* get_device_count (exla.cc:576-580) */
static ERL_NIF_TERM device_count(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  (void)argc; (void)argv;
  int n = 0, st = nxb200_init();
  if (st == NXB_OK) st = nxb200_device_count(&n);
  return st ? raise_status(env, st) : enif_make_int(env, n);
}

static ERL_NIF_TERM device_synchronize(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  int dev;
  if (argc != 1 || !enif_get_int(env, argv[0], &dev)) return BADARG(env);
  int st = nxb200_device_synchronize(dev);
  return st ? raise_status(env, st) : atom_ok;
}

/* ---- buffers -------------------------------------------------------------------------------------- */

/* binary_to_device_mem(device, type_code, shape, binary)   exla.cc:439-445, exla_client.cc:118-151 */
static ERL_NIF_TERM from_binary(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  int dev, dtype, rank;
  int64_t dims[NXB_MAX_RANK];
  ErlNifBinary bin;
  if (argc != 4 || !enif_get_int(env, argv[0], &dev) || !enif_get_int(env, argv[1], &dtype) ||
      !get_shape(env, argv[2], dims, &rank) || !enif_inspect_binary(env, argv[3], &bin))
    return BADARG(env);
  nxb200_buffer *b = NULL;
  /* the binary stays alive for the duration of this (dirty) call, which returns once the copy is done */
  int st = nxb200_buffer_from_host(dev, (nxb200_dtype)dtype, dims, rank, bin.data, bin.size, &b);
  return st ? raise_status(env, st) : wrap_buf(env, b);
}

/* read_device_mem(buffer, byte_limit)   exla.cc:447-453, exla_client.cc:58-72 */
static ERL_NIF_TERM to_binary(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  nxb200_buffer *b;
  ErlNifUInt64 limit;
  if (argc != 2 || !(b = get_buf(env, argv[0])) || !enif_get_uint64(env, argv[1], &limit)) return BADARG(env);
  ERL_NIF_TERM out;
  unsigned char *dst = enif_make_new_binary(env, (size_t)limit, &out);
  int st = nxb200_buffer_to_host(b, dst, (size_t)limit);
  return st ? raise_status(env, st) : out;
}

/* deallocate_device_mem   exla.cc:462-475 */
static ERL_NIF_TERM deallocate(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  nxb200_buffer *b;
  if (argc != 1 || !(b = get_buf(env, argv[0]))) return BADARG(env);
  int st = nxb200_buffer_deallocate(b);
  return st ? raise_status(env, st) : atom_ok;
}

/* is_device_buffer_deleted   exla.cc:477-482 */
static ERL_NIF_TERM is_deallocated(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  nxb200_buffer *b;
  int flag = 0;
  if (argc != 1 || !(b = get_buf(env, argv[0]))) return BADARG(env);
  int st = nxb200_buffer_is_deallocated(b, &flag);
  return st ? raise_status(env, st) : (flag ? atom_true : atom_false);
}

/* copy_buffer_to_device(buffer, device)   exla.cc:513-524 */
static ERL_NIF_TERM copy_to_device(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  nxb200_buffer *b, *out = NULL;
  int dev;
  if (argc != 2 || !(b = get_buf(env, argv[0])) || !enif_get_int(env, argv[1], &dev)) return BADARG(env);
  int st = nxb200_buffer_copy_to_device(b, dev, &out);
  return st ? raise_status(env, st) : wrap_buf(env, out);
}

/* get_buffer_typespec -> {type_code, shape, device}   exla.cc:455-460 */
static ERL_NIF_TERM buffer_info(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  nxb200_buffer *b;
  nxb200_dtype dt;
  int64_t dims[NXB_MAX_RANK];
  int rank, dev;
  if (argc != 1 || !(b = get_buf(env, argv[0]))) return BADARG(env);
  int st = nxb200_buffer_info(b, &dt, dims, &rank, &dev);
  if (st) return raise_status(env, st);
  return enif_make_tuple3(env, enif_make_int(env, (int)dt), make_shape(env, dims, rank), enif_make_int(env, dev));
}

/* get_buffer_device_pointer, :local mode -> address as an integer   exla.cc:325-389 */
static ERL_NIF_TERM device_pointer(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  nxb200_buffer *b;
  void *p = NULL;
  if (argc != 1 || !(b = get_buf(env, argv[0]))) return BADARG(env);
  int st = nxb200_buffer_device_pointer(b, &p);
  return st ? raise_status(env, st) : enif_make_uint64(env, (ErlNifUInt64)(uintptr_t)p);
}

/* create_buffer_from_device_pointer, :local mode   exla.cc:391-437 */
static ERL_NIF_TERM from_pointer(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  int dev, dtype, rank;
  int64_t dims[NXB_MAX_RANK];
  ErlNifUInt64 addr;
  if (argc != 4 || !enif_get_int(env, argv[0], &dev) || !enif_get_int(env, argv[1], &dtype) ||
      !get_shape(env, argv[2], dims, &rank) || !enif_get_uint64(env, argv[3], &addr))
    return BADARG(env);
  nxb200_buffer *b = NULL;
  int st = nxb200_buffer_from_pointer(dev, (nxb200_dtype)dtype, dims, rank, (void *)(uintptr_t)addr, &b);
  return st ? raise_status(env, st) : wrap_buf(env, b);
}

/* get_buffer_device_pointer, :cuda_ipc mode -> 64-byte handle binary */
static ERL_NIF_TERM ipc_export(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  nxb200_buffer *b;
  if (argc != 1 || !(b = get_buf(env, argv[0]))) return BADARG(env);
  ERL_NIF_TERM out;
  unsigned char *dst = enif_make_new_binary(env, NXB_IPC_HANDLE_BYTES, &out);
  int st = nxb200_buffer_ipc_export(b, dst);
  return st ? raise_status(env, st) : out;
}

/* create_buffer_from_device_pointer, :cuda_ipc mode */
static ERL_NIF_TERM from_ipc(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  int dev, dtype, rank;
  int64_t dims[NXB_MAX_RANK];
  ErlNifBinary h;
  if (argc != 4 || !enif_get_int(env, argv[0], &dev) || !enif_get_int(env, argv[1], &dtype) ||
      !get_shape(env, argv[2], dims, &rank) || !enif_inspect_binary(env, argv[3], &h) || h.size != NXB_IPC_HANDLE_BYTES)
    return BADARG(env);
  nxb200_buffer *b = NULL;
  int st = nxb200_buffer_from_ipc(dev, (nxb200_dtype)dtype, dims, rank, h.data, &b);
  return st ? raise_status(env, st) : wrap_buf(env, b);
}

/* buffer_alloc(device, type_code, shape): an uninitialised device tensor (outputs of program_run_into) */
static ERL_NIF_TERM buffer_alloc(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  int dev, dtype, rank;
  int64_t dims[NXB_MAX_RANK];
  if (argc != 3 || !enif_get_int(env, argv[0], &dev) || !enif_get_int(env, argv[1], &dtype) || !get_shape(env, argv[2], dims, &rank))
    return BADARG(env);
  nxb200_buffer *b = NULL;
  int st = nxb200_buffer_alloc(dev, (nxb200_dtype)dtype, dims, rank, &b);
  return st ? raise_status(env, st) : wrap_buf(env, b);
}

/* from_binary_async(device, type_code, shape, binary, pid, ref): the upload is queued and the call
 * returns; the binary is held in a private environment until the library has read its last byte, then
 * `{:nxb200_upload_done, ref}` is sent to `pid` and the environment is freed (exla_client.cc:118-151). */
typedef struct { ErlNifEnv *env; ErlNifPid to; ERL_NIF_TERM ref; } upload_ctx;

static void upload_done(void *p) {
  upload_ctx *u = p;
  ERL_NIF_TERM msg = enif_make_tuple2(u->env, enif_make_atom(u->env, "nxb200_upload_done"), u->ref);
  enif_send(NULL, &u->to, u->env, msg);      /* from a thread of the library: no calling environment */
  enif_free_env(u->env);                     /* releases the binary */
  enif_free(u);
}

static ERL_NIF_TERM from_binary_async(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  int dev, dtype, rank;
  int64_t dims[NXB_MAX_RANK];
  ErlNifBinary bin;
  upload_ctx *u;
  if (argc != 6 || !enif_get_int(env, argv[0], &dev) || !enif_get_int(env, argv[1], &dtype) || !get_shape(env, argv[2], dims, &rank))
    return BADARG(env);
  u = enif_alloc(sizeof *u);
  u->env = enif_alloc_env();
  ERL_NIF_TERM held = enif_make_copy(u->env, argv[3]);          /* refc binaries are shared, not copied */
  u->ref = enif_make_copy(u->env, argv[5]);
  if (!enif_get_local_pid(env, argv[4], &u->to) || !enif_inspect_binary(u->env, held, &bin)) {
    enif_free_env(u->env);
    enif_free(u);
    return BADARG(env);
  }
  nxb200_buffer *b = NULL;
  int st = nxb200_buffer_from_host_async(dev, (nxb200_dtype)dtype, dims, rank, bin.data, bin.size, upload_done, u, &b);
  if (st) {                                                     /* nothing was queued: the callback will not run */
    enif_free_env(u->env);
    enif_free(u);
    return raise_status(env, st);
  }
  return wrap_buf(env, b);
}

/* Transfers that complete at the next device_synchronize.  The host side of such a transfer is a
 * page-locked region owned by a resource (host_region), so that its address is stable and the BEAM
 * never sees it move; region_binary gives its bytes after the synchronisation. */
static ErlNifResourceType *HOST_TYPE;
typedef struct { void *ptr; size_t size; } host_res;
static void host_dtor(ErlNifEnv *env, void *p) { (void)env; host_res *r = p; if (r->ptr) enif_free(r->ptr); }

static ERL_NIF_TERM host_region(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  ErlNifUInt64 n;
  if (argc != 1 || !enif_get_uint64(env, argv[0], &n)) return BADARG(env);
  host_res *r = enif_alloc_resource(HOST_TYPE, sizeof *r);
  r->ptr = enif_alloc((size_t)n);          /* (a production build registers the pages with cudaHostRegister) */
  r->size = (size_t)n;
  ERL_NIF_TERM t = enif_make_resource(env, r);
  enif_release_resource(r);
  return t;
}

static ERL_NIF_TERM region_write(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  host_res *r;
  ErlNifBinary bin;
  if (argc != 2 || !enif_get_resource(env, argv[0], HOST_TYPE, (void **)&r) || !enif_inspect_binary(env, argv[1], &bin) || bin.size > r->size)
    return BADARG(env);
  memcpy(r->ptr, bin.data, bin.size);
  return atom_ok;
}

static ERL_NIF_TERM region_binary(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  host_res *r;
  if (argc != 1 || !enif_get_resource(env, argv[0], HOST_TYPE, (void **)&r)) return BADARG(env);
  return enif_make_resource_binary(env, r, r->ptr, r->size);
}

static ERL_NIF_TERM write_async(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  nxb200_buffer *b;
  host_res *r;
  ErlNifUInt64 n;
  if (argc != 3 || !(b = get_buf(env, argv[0])) || !enif_get_resource(env, argv[1], HOST_TYPE, (void **)&r) ||
      !enif_get_uint64(env, argv[2], &n) || n > r->size)
    return BADARG(env);
  int st = nxb200_buffer_write_async(b, r->ptr, (size_t)n);
  return st ? raise_status(env, st) : atom_ok;
}

static ERL_NIF_TERM read_async(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  nxb200_buffer *b;
  host_res *r;
  ErlNifUInt64 n;
  if (argc != 3 || !(b = get_buf(env, argv[0])) || !enif_get_resource(env, argv[1], HOST_TYPE, (void **)&r) ||
      !enif_get_uint64(env, argv[2], &n) || n > r->size)
    return BADARG(env);
  int st = nxb200_buffer_read_async(b, r->ptr, (size_t)n);
  return st ? raise_status(env, st) : atom_ok;
}

/* ---- programs ------------------------------------------------------------------------------------------ */

/* program_build(iodata): the serialised expression -> executable.  Replaces the thirteen MLIR builder
 * NIFs and mlir_compile (exla.cc:64-323). */
static ERL_NIF_TERM program_build(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  ErlNifBinary bin;
  if (argc != 1 || !enif_inspect_iolist_as_binary(env, argv[0], &bin)) return BADARG(env);
  nxb200_program *p = NULL;
  int st = nxb200_program_build(bin.data, bin.size, &p);
  if (st) return raise_status(env, st);
  prog_res *r = enif_alloc_resource(PROG_TYPE, sizeof *r);
  r->h = p;
  ERL_NIF_TERM t = enif_make_resource(env, r);
  enif_release_resource(r);
  return t;
}

/* [{type_code, shape}] of the results, what executable.ex:150-161 reads back */
static ERL_NIF_TERM program_outputs(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  nxb200_program *p;
  int n_in, n_out;
  if (argc != 1 || !(p = get_prog(env, argv[0]))) return BADARG(env);
  int st = nxb200_program_io(p, &n_in, &n_out);
  if (st) return raise_status(env, st);
  ERL_NIF_TERM list = enif_make_list(env, 0);
  for (int i = n_out - 1; i >= 0; --i) {
    nxb200_dtype dt;
    int64_t dims[NXB_MAX_RANK];
    int rank;
    if ((st = nxb200_program_output_info(p, i, &dt, dims, &rank))) return raise_status(env, st);
    list = enif_make_list_cell(env, enif_make_tuple2(env, enif_make_int(env, (int)dt), make_shape(env, dims, rank)), list);
  }
  return list;
}

/* run_io(program, device, [buffer]) -> [buffer]   exla.cc:626-634, exla_client.cc:258-398 */
static ERL_NIF_TERM program_run(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  nxb200_program *p;
  int dev, n_in, n_out;
  unsigned len;
  if (argc != 3 || !(p = get_prog(env, argv[0])) || !enif_get_int(env, argv[1], &dev) || !enif_get_list_length(env, argv[2], &len))
    return BADARG(env);
  int st = nxb200_program_io(p, &n_in, &n_out);
  if (st) return raise_status(env, st);
  nxb200_buffer **args = enif_alloc(sizeof(*args) * (len ? len : 1));
  nxb200_buffer **outs = enif_alloc(sizeof(*outs) * (n_out ? n_out : 1));
  ERL_NIF_TERM head, tail = argv[2];
  for (unsigned i = 0; i < len; ++i) {
    enif_get_list_cell(env, tail, &head, &tail);
    if (!(args[i] = get_buf(env, head))) { enif_free(args); enif_free(outs); return BADARG(env); }
  }
  st = nxb200_program_run(p, dev, args, (int)len, outs, n_out);
  ERL_NIF_TERM result;
  if (st) {
    result = raise_status(env, st);
  } else {
    result = enif_make_list(env, 0);
    for (int i = n_out - 1; i >= 0; --i) result = enif_make_list_cell(env, wrap_buf(env, outs[i]), result);
  }
  enif_free(args);
  enif_free(outs);
  return result;
}

/* human-readable plan (diagnostics) */
static ERL_NIF_TERM program_describe(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  nxb200_program *p;
  if (argc != 1 || !(p = get_prog(env, argv[0]))) return BADARG(env);
  size_t n = nxb200_program_describe(p, NULL, 0);
  char *tmp = enif_alloc(n + 1);
  nxb200_program_describe(p, tmp, n + 1);
  ERL_NIF_TERM out;
  memcpy(enif_make_new_binary(env, n, &out), tmp, n);
  enif_free(tmp);
  return out;
}

/* {plan_seconds, codegen_seconds}: the measurements of the compilation telemetry event */
static ERL_NIF_TERM program_build_times(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  nxb200_program *p;
  double a = 0, b = 0;
  if (argc != 1 || !(p = get_prog(env, argv[0]))) return BADARG(env);
  int st = nxb200_program_build_times(p, &a, &b);
  return st ? raise_status(env, st) : enif_make_tuple2(env, enif_make_double(env, a), enif_make_double(env, b));
}

/* program_run_into(program, device, [argument], [result]): results written into the given buffers */
static ERL_NIF_TERM program_run_into(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  nxb200_program *p;
  int dev;
  unsigned n_args, n_outs;
  if (argc != 4 || !(p = get_prog(env, argv[0])) || !enif_get_int(env, argv[1], &dev) || !enif_get_list_length(env, argv[2], &n_args) ||
      !enif_get_list_length(env, argv[3], &n_outs))
    return BADARG(env);
  nxb200_buffer **bufs = enif_alloc(sizeof(*bufs) * (n_args + n_outs + 1));
  ERL_NIF_TERM head, tail = argv[2];
  for (unsigned i = 0; i < n_args + n_outs; ++i) {
    if (i == n_args) tail = argv[3];
    enif_get_list_cell(env, tail, &head, &tail);
    if (!(bufs[i] = get_buf(env, head))) { enif_free(bufs); return BADARG(env); }
  }
  int st = nxb200_program_run_into(p, dev, bufs, (int)n_args, bufs + n_args, (int)n_outs);
  enif_free(bufs);
  return st ? raise_status(env, st) : atom_ok;
}

/* generated CUDA source of the i-th kernel (diagnostics); <<>> past the last one */
static ERL_NIF_TERM program_kernel_source(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  nxb200_program *p;
  int i;
  if (argc != 2 || !(p = get_prog(env, argv[0])) || !enif_get_int(env, argv[1], &i)) return BADARG(env);
  size_t n = nxb200_program_kernel_source(p, i, NULL, 0);
  char *tmp = enif_alloc(n + 1);
  nxb200_program_kernel_source(p, i, tmp, n + 1);
  ERL_NIF_TERM out;
  memcpy(enif_make_new_binary(env, n, &out), tmp, n);
  enif_free(tmp);
  return out;
}

static ERL_NIF_TERM program_launch_count(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  nxb200_program *p;
  int n = 0;
  if (argc != 1 || !(p = get_prog(env, argv[0]))) return BADARG(env);
  int st = nxb200_program_launch_count(p, &n);
  return st ? raise_status(env, st) : enif_make_int(env, n);
}

/* dot_bf16_static_scratch(device, a, b, c, m, n, k): the allocation-free product on three tensors of
 * the library, enqueued on the device's compute stream; complete on return */
static ERL_NIF_TERM dot_bf16_static_scratch(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  int dev;
  nxb200_buffer *a, *b, *c;
  ErlNifSInt64 m, n, k;
  void *pa, *pb, *pc, *stream;
  if (argc != 7 || !enif_get_int(env, argv[0], &dev) || !(a = get_buf(env, argv[1])) || !(b = get_buf(env, argv[2])) ||
      !(c = get_buf(env, argv[3])) || !enif_get_int64(env, argv[4], &m) || !enif_get_int64(env, argv[5], &n) || !enif_get_int64(env, argv[6], &k))
    return BADARG(env);
  int st = nxb200_buffer_device_pointer(a, &pa);
  if (!st) st = nxb200_buffer_device_pointer(b, &pb);
  if (!st) st = nxb200_buffer_device_pointer(c, &pc);
  if (!st) st = nxb200_device_stream(dev, &stream);
  if (!st) st = nxb200_dot_bf16_static_scratch(dev, pa, pb, pc, m, n, k, stream);
  return st ? raise_status(env, st) : atom_ok;
}

/* ---- device timing and self-test ---------------------------------------------------------------------- */

static ERL_NIF_TERM timer_begin(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  int dev;
  if (argc != 1 || !enif_get_int(env, argv[0], &dev)) return BADARG(env);
  int st = nxb200_timer_begin(dev);
  return st ? raise_status(env, st) : atom_ok;
}

static ERL_NIF_TERM timer_end(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  int dev;
  float ms = 0;
  if (argc != 1 || !enif_get_int(env, argv[0], &dev)) return BADARG(env);
  int st = nxb200_timer_end(dev, &ms);
  return st ? raise_status(env, st) : enif_make_double(env, ms);
}

/* the device's compute stream as an integer (for NIFs of other libraries that enqueue on it) */
static ERL_NIF_TERM device_stream(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  int dev;
  void *stream = NULL;
  if (argc != 1 || !enif_get_int(env, argv[0], &dev)) return BADARG(env);
  int st = nxb200_device_stream(dev, &stream);
  return st ? raise_status(env, st) : enif_make_uint64(env, (ErlNifUInt64)(uintptr_t)stream);
}

/* selftest_bounded_wait(device, limit_us) -> :timeout when the bounded wait gave up as it must */
static ERL_NIF_TERM selftest_bounded_wait(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  int dev;
  unsigned us;
  if (argc != 2 || !enif_get_int(env, argv[0], &dev) || !enif_get_uint(env, argv[1], &us)) return BADARG(env);
  int st = nxb200_selftest_bounded_wait(dev, us);
  if (st == NXB_ERR_TIMEOUT) return enif_make_atom(env, "timeout");
  return st ? raise_status(env, st) : atom_ok;
}

/* ---- memory counters (exla.cc:655-686) ---------------------------------------------------------------- */

static ERL_NIF_TERM memory_stats(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  int dev;
  uint64_t a, pk, r;
  if (argc != 1 || !enif_get_int(env, argv[0], &dev)) return BADARG(env);
  int st = nxb200_memory_stats(dev, &a, &pk, &r);
  if (st) return raise_status(env, st);
  return enif_make_tuple3(env, enif_make_uint64(env, a), enif_make_uint64(env, pk), enif_make_uint64(env, r));
}

static ERL_NIF_TERM memory_reset_peak(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  int dev;
  if (argc != 1 || !enif_get_int(env, argv[0], &dev)) return BADARG(env);
  int st = nxb200_memory_reset_peak(dev);
  return st ? raise_status(env, st) : atom_ok;
}

/* ---- sharded execution ------------------------------------------------------------------------------------ */

static ERL_NIF_TERM comm_id(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  (void)argc; (void)argv;
  ERL_NIF_TERM out;
  unsigned char *dst = enif_make_new_binary(env, NXB_COMM_ID_BYTES, &out);
  int st = nxb200_comm_id(dst);
  return st ? raise_status(env, st) : out;
}

static ERL_NIF_TERM comm_init(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  int dev, rank, world;
  ErlNifBinary id;
  if (argc != 4 || !enif_get_int(env, argv[0], &dev) || !enif_get_int(env, argv[1], &rank) || !enif_get_int(env, argv[2], &world) ||
      !enif_inspect_binary(env, argv[3], &id) || id.size != NXB_COMM_ID_BYTES)
    return BADARG(env);
  int st = nxb200_comm_init(dev, rank, world, id.data);
  return st ? raise_status(env, st) : atom_ok;
}

static ERL_NIF_TERM comm_peer_alloc(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  int dev;
  ErlNifUInt64 elems;
  if (argc != 2 || !enif_get_int(env, argv[0], &dev) || !enif_get_uint64(env, argv[1], &elems)) return BADARG(env);
  ERL_NIF_TERM out;
  unsigned char *dst = enif_make_new_binary(env, NXB_COMM_PEER_BLOB_BYTES, &out);
  int st = nxb200_comm_peer_alloc(dev, elems, dst);
  return st ? raise_status(env, st) : out;
}

static ERL_NIF_TERM comm_peer_open(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  ErlNifBinary blobs;
  int enabled = 0;
  if (argc != 1 || !enif_inspect_iolist_as_binary(env, argv[0], &blobs)) return BADARG(env);
  int st = nxb200_comm_peer_open(blobs.data, &enabled);
  return st ? raise_status(env, st) : (enabled ? atom_true : atom_false);
}

/* the sum over the group of one tensor, in place, on the compute stream (NCCL) */
static ERL_NIF_TERM comm_all_reduce_sum(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  nxb200_buffer *b;
  if (argc != 1 || !(b = get_buf(env, argv[0]))) return BADARG(env);
  int st = nxb200_comm_all_reduce_sum(b);
  return st ? raise_status(env, st) : atom_ok;
}

/* how many products ran fused with their exchange since the process started (diagnostics) */
static ERL_NIF_TERM comm_fused_launches(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  (void)argc; (void)argv;
  uint64_t n = 0;
  int st = nxb200_comm_fused_launches(&n);
  return st ? raise_status(env, st) : enif_make_uint64(env, n);
}

static ERL_NIF_TERM comm_destroy(ErlNifEnv *env, int argc, const ERL_NIF_TERM argv[]) {
  (void)argc; (void)argv;
  int st = nxb200_comm_destroy();
  return st ? raise_status(env, st) : atom_ok;
}

/* ---- module -------------------------------------------------------------------------------------------------- */

static int load(ErlNifEnv *env, void **priv, ERL_NIF_TERM info) {
  (void)priv; (void)info;
  ErlNifResourceFlags f = ERL_NIF_RT_CREATE | ERL_NIF_RT_TAKEOVER;
  BUF_TYPE = enif_open_resource_type(env, NULL, "nxb200_buffer", buf_dtor, f, NULL);
  PROG_TYPE = enif_open_resource_type(env, NULL, "nxb200_program", prog_dtor, f, NULL);
  HOST_TYPE = enif_open_resource_type(env, NULL, "nxb200_host_region", host_dtor, f, NULL);
  atom_ok = enif_make_atom(env, "ok");
  atom_error = enif_make_atom(env, "error");
  atom_already_deallocated = enif_make_atom(env, "already_deallocated");
  atom_true = enif_make_atom(env, "true");
  atom_false = enif_make_atom(env, "false");
  return BUF_TYPE && PROG_TYPE && HOST_TYPE ? 0 : -1;
}

static ErlNifFunc funcs[] = {
    {"device_count", 0, device_count, 0},
    {"device_synchronize", 1, device_synchronize, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"from_binary", 4, from_binary, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"to_binary", 2, to_binary, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"deallocate", 1, deallocate, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"is_deallocated", 1, is_deallocated, 0},
    {"copy_to_device", 2, copy_to_device, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"buffer_info", 1, buffer_info, 0},
    {"device_pointer", 1, device_pointer, 0},
    {"from_pointer", 4, from_pointer, 0},
    {"ipc_export", 1, ipc_export, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"from_ipc", 4, from_ipc, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"buffer_alloc", 3, buffer_alloc, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"from_binary_async", 6, from_binary_async, 0},
    {"host_region", 1, host_region, 0},
    {"region_write", 2, region_write, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"region_binary", 1, region_binary, 0},
    {"write_async", 3, write_async, 0},
    {"read_async", 3, read_async, 0},
    {"program_build", 1, program_build, ERL_NIF_DIRTY_JOB_CPU_BOUND},
    {"program_outputs", 1, program_outputs, 0},
    {"program_run", 3, program_run, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"program_describe", 1, program_describe, 0},
    {"program_build_times", 1, program_build_times, 0},
    {"program_run_into", 4, program_run_into, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"program_kernel_source", 2, program_kernel_source, 0},
    {"program_launch_count", 1, program_launch_count, 0},
    {"dot_bf16_static_scratch", 7, dot_bf16_static_scratch, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"timer_begin", 1, timer_begin, 0},
    {"timer_end", 1, timer_end, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"device_stream", 1, device_stream, 0},
    {"selftest_bounded_wait", 2, selftest_bounded_wait, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"memory_stats", 1, memory_stats, 0},
    {"memory_reset_peak", 1, memory_reset_peak, 0},
    {"comm_id", 0, comm_id, 0},
    {"comm_init", 4, comm_init, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"comm_peer_alloc", 2, comm_peer_alloc, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"comm_peer_open", 1, comm_peer_open, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"comm_all_reduce_sum", 1, comm_all_reduce_sum, ERL_NIF_DIRTY_JOB_IO_BOUND},
    {"comm_fused_launches", 0, comm_fused_launches, 0},
    {"comm_destroy", 0, comm_destroy, ERL_NIF_DIRTY_JOB_IO_BOUND},
};

ERL_NIF_INIT(Elixir.NxB200.NIF, funcs, load, NULL, NULL, NULL)
