"""ctypes binding of include/tagi_b200_comm.h (libtagi_b200_comm.so) and a small data-parallel helper on top of it."""
import ctypes as C
import os

from .capi import TagiError

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtagi_b200_comm.so")
ID_BYTES = 128
_lib = None

_p, _i, _z = C.c_void_p, C.c_int, C.c_size_t
_SIG = {
    "tagi_rendezvous_publish": [C.c_char_p, _p, _z],
    "tagi_rendezvous_fetch": [C.c_char_p, _p, _z, _i],
    "tagi_rendezvous_publish_id": [C.c_char_p, _p, _i],
    "tagi_rendezvous_fetch_id": [C.c_char_p, _p, _i, _i],
    "tagi_comm_plan_buckets": [C.POINTER(_z), _i, _z, C.POINTER(_i)],
    "tagi_comm_create_id": [_p],
    "tagi_comm_init": [_p, _i, _i, _i],
    "tagi_comm_init_file": [C.c_char_p, _i, _i, _i, _i],
    "tagi_comm_rank": [],
    "tagi_comm_world_size": [],
    "tagi_comm_register": [_p, _z],
    "tagi_comm_finalize_buckets": [_z],
    "tagi_comm_num_buckets": [],
    "tagi_comm_num_tensors": [],
    "tagi_comm_num_collectives": [],
    "tagi_comm_bucket_of": [_i],
    "tagi_comm_tensor_ready": [_i, _p, _i],
    "tagi_comm_flush": [_p, _i],
    "tagi_comm_wait": [_p],
    "tagi_comm_allreduce": [_p, _z, _i, _p],
    "tagi_comm_broadcast": [_p, _z, _i, _p],
    "tagi_comm_check": [],
    "tagi_comm_barrier": [],
    "tagi_comm_sync_stream": [],
    "tagi_comm_set_max_ctas": [_i],
    "tagi_comm_destroy": [],
}
_RAW = {"tagi_comm_rank", "tagi_comm_world_size", "tagi_comm_num_buckets", "tagi_comm_num_tensors", "tagi_comm_num_collectives",
        "tagi_comm_bucket_of",
        "tagi_comm_plan_buckets", "tagi_comm_register"}


def _preload_nccl():
    """A process has room for one libnccl.so.2. PyTorch ships its own (newer than the system copy this library was linked
    against) and fails to import if an older one is already resident, so when that copy exists it is loaded first and
    this library binds to it."""
    try:
        import importlib.util
        spec = importlib.util.find_spec("nvidia.nccl")
        if spec and spec.submodule_search_locations:
            cand = os.path.join(list(spec.submodule_search_locations)[0], "lib", "libnccl.so.2")
            if os.path.exists(cand):
                C.CDLL(cand, mode=C.RTLD_GLOBAL)
    except (ImportError, OSError, ValueError):
        pass


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} not found: run python -m cutagi_b200.build")
        _preload_nccl()
        _lib = C.CDLL(LIB_PATH)
        _lib.tagi_comm_last_error_string.restype = C.c_char_p
        for n, a in _SIG.items():
            f = getattr(_lib, n)
            f.argtypes, f.restype = a, _i
    return _lib


def _call(name, *args):
    rc = getattr(load(), name)(*args)
    if name in _RAW:
        if rc < 0:
            raise TagiError(-rc, load().tagi_comm_last_error_string().decode())
        return rc
    if rc != 0:
        raise TagiError(rc, load().tagi_comm_last_error_string().decode())
    return rc


def rendezvous_publish(path, blob: bytes):
    _call("tagi_rendezvous_publish", path.encode(), blob, len(blob))


def rendezvous_fetch(path, nbytes, timeout_ms):
    buf = C.create_string_buffer(nbytes)
    _call("tagi_rendezvous_fetch", path.encode(), buf, nbytes, timeout_ms)
    return buf.raw


def rendezvous_publish_id(path, ident: bytes, world_size):
    assert len(ident) == ID_BYTES
    _call("tagi_rendezvous_publish_id", path.encode(), ident, world_size)


def rendezvous_fetch_id(path, world_size, timeout_ms):
    buf = C.create_string_buffer(ID_BYTES)
    _call("tagi_rendezvous_fetch_id", path.encode(), buf, world_size, timeout_ms)
    return buf.raw


def plan_buckets(counts, bucket_bytes):
    """Bucket index of every tensor (greedy packing in registration order) and the number of buckets."""
    n = len(counts)
    arr = (_z * n)(*counts)
    out = (_i * n)()
    nb = _call("tagi_comm_plan_buckets", arr, n, bucket_bytes, out)
    return list(out), nb


class DeltaExchange:
    """Bucketed, overlapped allreduce of parameter-delta tensors over NCCL (one instance per process).

    tensors: CUDA float32 tensors in the order their backward passes produce them.
    """

    def __init__(self, tensors, rank, world_size, device, rendezvous_path, bucket_bytes=32 << 20, average=True,
                 timeout_ms=60000, max_ctas=0):
        self.average = int(average)
        if max_ctas:
            _call("tagi_comm_set_max_ctas", max_ctas)
        _call("tagi_comm_init_file", rendezvous_path.encode(), rank, world_size, device, timeout_ms)
        self.index = [_call("tagi_comm_register", t.data_ptr(), t.numel()) for t in tensors]
        _call("tagi_comm_finalize_buckets", bucket_bytes)
        self.num_buckets = load().tagi_comm_num_buckets()
        self.num_collectives = load().tagi_comm_num_collectives()   # fewer than tensors when adjacent ones were merged

    def ready(self, i, stream_ptr):
        _call("tagi_comm_tensor_ready", self.index[i], stream_ptr, self.average)

    def flush(self, stream_ptr):
        _call("tagi_comm_flush", stream_ptr, self.average)

    def wait(self, stream_ptr):
        _call("tagi_comm_wait", stream_ptr)

    def broadcast(self, t, root, stream_ptr):
        _call("tagi_comm_broadcast", t.data_ptr(), t.numel(), root, stream_ptr)

    def check(self):
        _call("tagi_comm_check")

    def barrier(self):
        _call("tagi_comm_barrier")

    def allreduce(self, t, stream_ptr, average=None):
        _call("tagi_comm_allreduce", t.data_ptr(), t.numel(), self.average if average is None else int(average),
              stream_ptr)

    def close(self):
        _call("tagi_comm_destroy")
