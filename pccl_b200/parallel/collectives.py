"""Collectives on top of the engine: pick an algorithm, compile the plan once,
register it, run it.

    import pccl_b200.parallel as pp
    pp.init(group)                               # connects the engine
    x = pp.working_tensor(n, torch.float32)      # lives in the symmetric heap
    pp.all_reduce(x)                             # in place, no staging copies

Plans are cached per (collective, algorithm, world, dtype, numel, channels).  The
algorithm comes from ``select_algorithm`` with the B200 profile unless given (or
forced with ``PCCL_ALGO``); ``PCCL_CHANNELS`` overrides the channel count.

The reference has no such layer: its benchmarks build a template, compile it to
a file and call register/execute by hand (tests/bench_algo_comparison.py:60-121).
"""

from __future__ import annotations

import os
import tempfile
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from .. import engine as _engine
from ..dsl.algorithms import ALGORITHMS, select_algorithm
from ..dsl.algorithms.selector import tuned_route
from ..dsl.compiler import Compiler
from ..dsl.superopt.cost_model import B200_PROFILE, NVLINK5_TOPOLOGY, TopologyProfile

_DTYPE_NAME = {torch.float32: "float32", torch.float16: "float16", torch.bfloat16: "bfloat16"}
for _name, _plan_name in (("float8_e4m3fn", "float8_e4m3"), ("float8_e5m2", "float8_e5m2")):
    if hasattr(torch, _name):
        _DTYPE_NAME[getattr(torch, _name)] = _plan_name

_state: Dict[str, object] = {"group": None, "rank": 0, "world": 1, "registered": {}, "dir": None}


def init(group: Optional[dist.ProcessGroup] = None):
    """Connect the engine over ``group`` (default group when None).  Collective; a second call with the
    engine already connected returns it without allocating anything again."""
    if _state.get("connected"):
        return _engine.get_engine()
    _state["group"] = group
    if dist.is_initialized():
        _state["rank"], _state["world"] = dist.get_rank(group), dist.get_world_size(group)
    os.environ.setdefault("RANK", str(_state["rank"]))
    os.environ.setdefault("WORLD_SIZE", str(_state["world"]))
    if dist.is_initialized():
        _engine.initialize_engine(group)
    else:
        _engine.get_engine()
    # Error words of this layer's fused kernels: [0] packet all-reduce, [1] push collectives.  Each
    # kernel family aborts on its own word only, so one timeout does not poison the others.
    _state["errors"] = torch.zeros(4, dtype=torch.int32, device="cuda") if torch.cuda.is_available() \
        and os.environ.get("PCCL_EXECUTOR") != "cpu" else None
    _state["err_ll"] = _state["errors"][0:1] if _state["errors"] is not None else None
    _state["err_push"] = _state["errors"][1:2] if _state["errors"] is not None else None
    _state["err_nvls"] = _state["errors"][2:3] if _state["errors"] is not None else None
    _setup_ll(group)
    _setup_push(group)
    _setup_nvls(group)
    _state["connected"] = True
    return _engine.get_engine()


#: largest message (bytes) the packet-protocol all-reduce takes.  Its payload doubles on the wire and
#: every rank sends to every peer, so the default shrinks with the world size: 4 MB / world
#: (2 MB for two ranks, 512 KB for eight); PCCL_LL_MAX_BYTES overrides it.
LL_MAX_BYTES = 256 << 10


def _ll_limit(world: int) -> int:
    forced = os.environ.get("PCCL_LL_MAX_BYTES")
    if forced:
        from ..config import _size
        return _size(forced)
    return (4 << 20) // max(2, world)


def _setup_ll(group) -> None:
    """Receive buffer of the small-message all-reduce: [2 parities][world][2 x LL_MAX_BYTES], zeroed."""
    global LL_MAX_BYTES
    eng = _engine.get_engine()
    _state["ll"] = None
    LL_MAX_BYTES = _ll_limit(_state["world"])
    if _state["world"] < 2 or not torch.cuda.is_available() or not hasattr(eng, "empty_symmetric") \
            or LL_MAX_BYTES <= 0 or os.environ.get("PCCL_EXECUTOR") == "cpu":
        return
    buf = eng.empty_symmetric((2 * _state["world"] * 2 * LL_MAX_BYTES,), torch.uint8)
    buf.zero_()
    torch.cuda.synchronize()
    dist.barrier(group=group)
    _state["ll"] = {"buf": buf, "epoch": 0, "native": _engine.load_native().fused}


#: largest message (bytes) taken by the fused push all-reduce (PCCL_PUSH_MAX_BYTES); larger ones run as
#: plans, zero-copy on symmetric tensors
PUSH_MAX_BYTES = 32 << 20
_PUSH_CTAS = 96


def _setup_push(group) -> None:
    """Receive areas of the push all-reduce: [2 parities][A | B][world][slot], flags, counters."""
    global PUSH_MAX_BYTES
    _state["push"] = None
    forced = os.environ.get("PCCL_PUSH_MAX_BYTES")
    if forced:
        from ..config import _size
        PUSH_MAX_BYTES = _size(forced)
    eng = _engine.get_engine()
    world = _state["world"]
    if world < 2 or not torch.cuda.is_available() or not hasattr(eng, "empty_symmetric") \
            or PUSH_MAX_BYTES <= 0 or os.environ.get("PCCL_EXECUTOR") == "cpu":
        return
    slot = ((PUSH_MAX_BYTES // 16 + world - 1) // world) * 16
    areas = eng.empty_symmetric((4 * world * slot,), torch.uint8)
    flags = eng.empty_symmetric((2 * world,), torch.int32)
    flags.zero_()
    torch.cuda.synchronize()
    dist.barrier(group=group)
    _state["push"] = {"areas": areas, "flags": flags, "epoch": 0, "native": _engine.load_native().fused,
                      "counters": torch.zeros(2, dtype=torch.int32, device="cuda")}


def ensure_lean_push(ctas: Optional[int] = None) -> bool:
    """A second instance of the push kernel's buffers, run with few CTAs (``PCCL_PUSH_LEAN_CTAS``, default
    12): for collectives that should hide under compute kernels (``all_reduce(..., overlap=True)``), where
    a grid of 96 CTAs would take two thirds of the SMs from the GEMM it runs beside.  Posted NVLink stores
    keep the link busy from a few hundred warps, so the lean grid loses little bandwidth.  Collective (it
    allocates symmetric memory): every rank calls it at the same point.  True when the instance exists."""
    if _state.get("push_lean") is not None:
        return True
    main = _state.get("push")
    if main is None:
        return False
    eng = _engine.get_engine()
    world = _state["world"]
    slot = ((PUSH_MAX_BYTES // 16 + world - 1) // world) * 16
    try:
        areas = eng.empty_symmetric((4 * world * slot,), torch.uint8)
        flags = eng.empty_symmetric((2 * world,), torch.int32)
    except RuntimeError:
        # The symmetric arena is full (the same on every rank: they allocate alike): overlapped calls
        # then share the main instance.
        return False
    flags.zero_()
    torch.cuda.synchronize()
    dist.barrier(group=_state["group"])
    _state["push_lean"] = {"areas": areas, "flags": flags, "epoch": 0, "native": main["native"],
                           "counters": torch.zeros(2, dtype=torch.int32, device="cuda"),
                           "ctas": int(ctas or os.environ.get("PCCL_PUSH_LEAN_CTAS", "12"))}
    return True


_NVLS_DTYPE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _setup_nvls(group) -> None:
    """Flags and counter of the in-switch all-reduce kernel (algorithm "nvls_kernel")."""
    _state["nvls"] = None
    eng = _engine.get_engine()
    if _state["world"] < 2 or not torch.cuda.is_available() or not hasattr(eng, "empty_symmetric") \
            or os.environ.get("PCCL_EXECUTOR") == "cpu" or not eng.nvls_active():
        return
    flags = eng.empty_symmetric((2 * _state["world"],), torch.int32)
    flags.zero_()
    torch.cuda.synchronize()
    dist.barrier(group=group)
    _state["nvls"] = {"flags": flags, "epoch": 0, "native": _engine.load_native().fused,
                      "counter": torch.zeros(1, dtype=torch.int32, device="cuda"),
                      "ctas": max(1, int(os.environ.get("PCCL_NVLS_CTAS", "64")))}


def _nvls_kernel_ok(tensor: torch.Tensor, op: str) -> bool:
    """Sizes, dtype and arguments only (the same answer on every rank); where the tensor lives decides
    staging, never the path."""
    nbytes = tensor.numel() * tensor.element_size()
    return (_state.get("nvls") is not None and op == "sum" and tensor.is_cuda and tensor.dtype in _NVLS_DTYPE
            and nbytes > 0 and nbytes % (16 * _state["world"]) == 0)


def _is_symmetric(tensor: torch.Tensor) -> bool:
    eng = _engine.get_engine()
    native = getattr(eng, "native", None)
    return bool(tensor.is_cuda and tensor.is_contiguous() and native is not None
                and native.heapOffset(tensor) >= 0 and native.heapOffset(tensor) % 16 == 0)


def _nvls_kernel(tensor: torch.Tensor) -> None:
    """In-switch all-reduce of `tensor`, in place when it lies in symmetric memory, else through the
    working buffer (two device copies more)."""
    nv = _state["nvls"]
    eng = _engine.get_engine()
    nbytes = tensor.numel() * tensor.element_size()
    offset = eng.native.heapOffset(tensor) if tensor.is_contiguous() else -1
    staged = None
    if offset < 0 or offset % 16:
        staged = eng.working_buffer(tensor.numel(), tensor.dtype)
        staged.copy_(tensor.reshape(-1))
        offset = 0
    nv["epoch"] += 1
    nv["native"].allreduce_nvls(offset, nbytes, _NVLS_DTYPE[tensor.dtype], nv["flags"].heap_offset, nv["counter"],
                                nv["epoch"], nv["ctas"], _state["err_nvls"])
    if staged is not None:
        tensor.copy_(staged.view_as(tensor) if tensor.is_contiguous() else staged.reshape(tensor.shape))


def _push_eligible(tensor: torch.Tensor, op: str, algorithm: Optional[str]) -> bool:
    """Sizes, dtype and arguments only: the same answer on every rank whatever view each rank passes.
    A view that the kernel cannot take directly (not contiguous, not 16-byte aligned) is staged through
    an aligned copy by ``_aligned``; it never changes which kernel runs."""
    push = _state.get("push")
    if push is None or op != "sum" or algorithm not in (None, "push"):
        return False
    nbytes = tensor.numel() * tensor.element_size()
    return (tensor.is_cuda and nbytes % 16 == 0 and 0 < nbytes <= PUSH_MAX_BYTES
            and tensor.dtype in (torch.float32, torch.float16, torch.bfloat16))


def _aligned(tensor: torch.Tensor, align: int = 16) -> torch.Tensor:
    """``tensor`` itself when a kernel can read it in place, else a contiguous, aligned copy of it
    (fresh allocations are at least 256-byte aligned)."""
    if tensor.is_contiguous() and tensor.data_ptr() % align == 0:
        return tensor
    return tensor.contiguous().clone() if tensor.is_contiguous() else tensor.contiguous()


def _push(mode: int, input: torch.Tensor, output: torch.Tensor, lean: bool = False) -> None:
    push = _state["push_lean"] if lean else _state["push"]
    push["epoch"] += 1
    src, dst = _aligned(input), _aligned(output)
    if mode == 0 and input.data_ptr() == output.data_ptr() and src is not input:
        dst = src                                  # in place on the staged copy
    push["native"].collective_push(mode, src, dst, push["areas"].heap_offset, PUSH_MAX_BYTES,
                                   push["flags"].heap_offset, push["counters"], push["epoch"],
                                   push.get("ctas", _PUSH_CTAS), _state["err_push"])
    if dst is not output:
        output.copy_(dst)


def _push_ok(full: torch.Tensor, part: torch.Tensor, algorithm: Optional[str], executor: Optional[str] = None,
             op: str = "sum") -> bool:
    """Reduce-scatter / all-gather / all-to-all through the push kernel: `full` is the whole message.

    The answer depends only on things that are the same on every rank (sizes, dtype, arguments); the part
    may be this rank's slice of `full` (the in-place conventions of all-gather and reduce-scatter)."""
    if _state.get("push") is None or algorithm not in (None, "push") or executor is not None or op != "sum":
        return False
    world = _state["world"]
    nbytes = full.numel() * full.element_size()
    return (full.is_cuda and part.is_cuda
            and full.dtype == part.dtype and full.dtype in (torch.float32, torch.float16, torch.bfloat16)
            and 0 < nbytes <= PUSH_MAX_BYTES and nbytes % (16 * world) == 0)


def _ll_eligible(tensor: torch.Tensor, op: str, algorithm: Optional[str]) -> bool:
    ll = _state.get("ll")
    if ll is None or op != "sum" or algorithm not in (None, "ll"):
        return False
    nbytes = tensor.numel() * tensor.element_size()
    return (tensor.is_cuda and nbytes % 8 == 0 and 0 < nbytes <= LL_MAX_BYTES
            and tensor.dtype in (torch.float32, torch.float16, torch.bfloat16))


_shard_route_cache: Dict[Tuple[str, int], Optional[str]] = {}


def _routed_shard_kernel(kind: str, full_bytes: int) -> Optional[str]:
    """"ll" / "push" when the measured table names that kernel for this collective and size, else None."""
    key = (kind, full_bytes)
    if key not in _shard_route_cache:
        route = None if os.environ.get("PCCL_ALGO") else tuned_route(kind, _state["world"], full_bytes)
        _shard_route_cache[key] = route["algorithm"] if route and route["algorithm"] in ("ll", "push") else None
    return _shard_route_cache[key]


def _ll_part_ok(part: torch.Tensor, full: torch.Tensor, algorithm: Optional[str], executor: Optional[str] = None,
                op: str = "sum", kind: Optional[str] = None) -> bool:
    """Reduce-scatter / all-gather / all-to-all through the packet kernel: `part` is what one rank sends
    to (or receives from) one peer.  Sizes, dtype and arguments only.  Unforced, the measured table
    decides where it names a kernel for this size; without one the packet kernel takes parts of up to
    half its buffer.  ``algorithm="ll"`` takes what fits."""
    ll = _state.get("ll")
    if ll is None or op != "sum" or algorithm not in (None, "ll") or executor is not None:
        return False
    nbytes = part.numel() * part.element_size()
    limit = LL_MAX_BYTES if algorithm == "ll" else LL_MAX_BYTES // 2
    if algorithm is None and kind is not None:
        routed = _routed_shard_kernel(kind, full.numel() * full.element_size())
        if routed == "push":
            return False
        if routed == "ll":
            limit = LL_MAX_BYTES
    return (part.is_cuda and full.is_cuda and part.dtype == full.dtype and nbytes % 8 == 0 and 0 < nbytes <= limit
            and part.dtype in (torch.float32, torch.float16, torch.bfloat16))


def _ll_collective(mode: int, input: torch.Tensor, output: torch.Tensor) -> None:
    ll = _state["ll"]
    ll["epoch"] += 1
    src, dst = _aligned(input, 8), _aligned(output, 8)
    ll["native"].collective_ll(mode, src, dst, ll["buf"].heap_offset, LL_MAX_BYTES, ll["epoch"], _state["err_ll"])
    if dst is not output:
        output.copy_(dst)


def working_tensor(shape, dtype=torch.float32) -> torch.Tensor:
    """Tensor that aliases the engine's working buffer (offset 0)."""
    return _engine.working_buffer(shape, dtype)


def _topology() -> TopologyProfile:
    nvls = getattr(_engine.get_engine(), "nvls_active", lambda: False)()
    return NVLINK5_TOPOLOGY if nvls else TopologyProfile("nvlink5", 900.0, 0.7, uniform_all_to_all=True)


def default_channels(nbytes: int, world: int) -> int:
    forced = os.environ.get("PCCL_CHANNELS")
    if forced:
        return max(1, int(forced))
    # One channel per ~8 MiB so that the reduce half of channel c+1 overlaps the gather half of c.
    return max(1, min(16, nbytes // (8 << 20)))


def _plan_name(kind: str, algorithm: str, dtype: str, numel: int, channels: int) -> str:
    return f"{kind}_{algorithm}_{dtype}_{numel}_c{channels}_w{_state['world']}"


def ensure_plan(kind: str, numel: int, dtype: torch.dtype, algorithm: Optional[str] = None,
                channels: Optional[int] = None, reduce_op: str = "sum", executor: Optional[str] = None) -> str:
    """Compile + register (once) the plan for this collective; returns its name."""
    world, rank = _state["world"], _state["rank"]
    dtype_name = _DTYPE_NAME[dtype]
    nbytes = numel * torch.empty((), dtype=dtype).element_size()
    if algorithm is None:
        algorithm = os.environ.get("PCCL_ALGO")
    if algorithm is None:
        if kind == "allreduce":
            algorithm = select_algorithm(world, nbytes, _topology(), B200_PROFILE).name
        else:
            # The measured table first.  Without one: direct pulls.  In-switch multicast does not lower
            # the busier direction of an all-gather or reduce-scatter (each rank still receives, or
            # serves, (W-1)/W of the message), and peer loads moved 650 GB/s against 571 GB/s for
            # multimem on 4 GPUs.
            route = tuned_route(kind, world, nbytes) if kind in ("allgather", "reduce_scatter") else None
            algorithm = route["algorithm"] if route and route["algorithm"] in ALGORITHMS else "twoshot"
            if route and route["algorithm"] in ALGORITHMS and channels is None:
                channels = route.get("channels")
    if channels is None:
        channels = default_channels(nbytes, world)
    if algorithm in ("ring", "rhd", "tree") and kind != "allreduce":
        # The reference-compatible ring templates interleave channels inside the tensor, which
        # does not match the contiguous shard the engine reads / writes for these collectives.
        channels = 1
    # Every channel's slice must split evenly over the ranks, in 16-byte units where possible.
    if algorithm == "hybrid":
        channels = max(2, channels)              # at least one in-switch and one peer channel; it rounds by itself
    else:
        while channels > 1 and numel % (channels * world):
            channels //= 2
    name = _plan_name(kind, algorithm, dtype_name, numel, channels) + ("" if reduce_op == "sum" else "_" + reduce_op) \
        + ("" if executor in (None, "sm") else "_" + executor)
    if algorithm == "hybrid":
        name += "_f" + os.environ.get("PCCL_NVLS_FRACTION", "0.7")
    if name in _state["registered"]:
        return name
    plan_executor = executor or ("multimem" if algorithm in ("nvls", "nvls_twopass", "hybrid") else "sm")

    def compile_for(r: int) -> str:
        graph = getattr(ALGORITHMS[algorithm](), "build_" + kind)(r, world, numel, dtype_name, plan_executor, channels)
        if reduce_op != "sum":
            for node in graph.nodes.values():
                if hasattr(node, "reduce_op"):
                    node.reduce_op = reduce_op
        return Compiler().compile_to_json(graph)

    text = _plan_from_cache(name, rank, world, compile_for)
    engine = _engine.get_engine()
    if hasattr(engine, "register_operation_from_string"):
        ok = engine.register_operation_from_string(name, text)
    else:
        if _state["dir"] is None:
            _state["dir"] = tempfile.mkdtemp(prefix="pccl-plans-")
        path = os.path.join(_state["dir"], name + ".json")
        with open(path, "w") as handle:
            handle.write(text)
        ok = engine.register_operation(name, path)
    if not ok:
        raise _engine.PCCLError(f"could not register plan '{name}'")
    if dist.is_initialized() and world > 1:
        dist.barrier(group=_state["group"])      # nobody signals a rank that has not registered yet
    _state["registered"][name] = (kind, algorithm, channels)
    return name


_route_cache: Dict[int, Tuple[Optional[str], Optional[int]]] = {}


def _routed_allreduce(nbytes: int) -> Tuple[Optional[str], Optional[int]]:
    """(algorithm, channels) the tuning file names for an all-reduce of this size, or (None, None)."""
    if os.environ.get("PCCL_ALGO") is not None:
        return None, None
    route = tuned_route("allreduce", _state["world"], nbytes)
    if route is None:
        return None, None
    choice = route["algorithm"]
    if choice in ("ll", "push", "nvls_kernel") or choice in ALGORITHMS:
        return choice, route.get("channels")
    return None, None


def _plan_cache_dir() -> Optional[str]:
    where = os.environ.get("PCCL_PLAN_CACHE", os.path.expanduser("~/.pccl/plans"))
    return None if where.lower() in ("", "0", "off", "none") else where


def _plan_from_cache(name: str, rank: int, world: int, compile_for) -> str:
    """This rank's compiled plan: from the on-disk cache when the same (collective, algorithm, dtype,
    size, channels, world, rank, library version) was compiled before, else compiled now, and, before
    it is stored, checked together with every other rank's plan: the engine's abstract replay of the
    signal protocol (``PCCL_VALIDATE=0`` skips it) refuses a set that would deadlock or leave signals
    behind.  Templates are deterministic, so every rank can build all ranks' plans without talking
    to anyone; a cached plan was checked when it was first compiled."""
    import hashlib
    from .. import __version__
    where = _plan_cache_dir()
    extra = os.environ.get("PCCL_NVLS_FRACTION", "") if "hybrid" in name else ""
    key = hashlib.sha1(f"{name}|rank{rank}|{__version__}|{extra}".encode()).hexdigest()
    path = os.path.join(where, key + ".json") if where else None
    if path and os.path.exists(path):
        try:
            with open(path) as handle:
                text = handle.read()
            if text.lstrip().startswith("{"):
                return text
        except OSError:
            pass
    text = compile_for(rank)
    if os.environ.get("PCCL_VALIDATE", "1") != "0" and world > 1 and not isinstance(_engine.get_engine(), _engine.CpuEngine):
        native = _engine.load_native()
        report = native.check_world([text if r == rank else compile_for(r) for r in range(world)])
        if report["deadlock"] or report["leftover_signals"]:
            raise _engine.PCCLError(f"plan '{name}' fails the signal-protocol check: {report['detail']}")
    if path:
        try:
            os.makedirs(where, exist_ok=True)
            tmp = f"{path}.{os.getpid()}.tmp"
            with open(tmp, "w") as handle:
                handle.write(text)
            os.replace(tmp, path)
        except OSError:
            pass
    return text


def all_reduce(tensor: torch.Tensor, op: str = "sum", algorithm: Optional[str] = None,
               channels: Optional[int] = None, async_op: bool = False, overlap: bool = False) -> torch.Tensor:
    """In-place all-reduce of ``tensor`` (sum / max / min / avg).

    ``overlap=True`` says the call runs beside compute kernels (gradient buckets under backward): sums
    that fit the push kernel then run on its lean instance (see ``ensure_lean_push``), whatever the
    table says is fastest on an idle GPU.

    Unless an algorithm is forced, the measured table for this world size picks the path: the
    packet-protocol kernel (small sums), the fused push kernel (up to ``PUSH_MAX_BYTES``), the in-switch
    kernel (tensors in symmetric memory, and anything above the push kernel's range when NVLS is up) or
    a plan.  Without a table: packet kernel up to ``LL_MAX_BYTES``, push kernel up to ``PUSH_MAX_BYTES``,
    then plans.  The kernels are asynchronous on the current stream and need no staging copy (the
    in-switch kernel stages ordinary tensors through the working buffer).  An average is the same sum
    followed by a scale.
    """
    if op == "avg" and algorithm in (None, "ll", "push", "nvls_kernel") and tensor.dtype in _NVLS_DTYPE \
            and (_state.get("ll") or _state.get("push") or _state.get("nvls")):
        # The fused kernels sum; the average is the sum times 1 / world (one element-wise pass, as the
        # plans' own avg does).  Which kernel runs is decided exactly as for a sum.
        all_reduce(tensor, "sum", algorithm, channels, async_op=True, overlap=overlap)
        tensor.mul_(1.0 / _state["world"])
        if not async_op:
            synchronize()
        return tensor
    if overlap and algorithm is None and _state.get("push_lean") is not None and _push_eligible(tensor, op, None):
        _push(0, tensor, tensor, lean=True)
        return tensor
    if algorithm is None and op == "sum":
        # A measured table, when one covers this world size, says which path wins at this size
        # (same file on every rank, so every rank takes the same path).  Looked up once per size.
        nbytes = tensor.numel() * tensor.element_size()
        routed = _route_cache.get(nbytes)
        if routed is None:
            routed = _route_cache[nbytes] = _routed_allreduce(nbytes)
        if routed[0] == "nvls_kernel":
            # The table is measured in place on symmetric tensors.  An ordinary tensor would be staged
            # through the working buffer (two copies more), which only pays above the push kernel's
            # range.  Where a tensor lives is the same on every rank by construction: symmetric
            # allocations are collective calls.
            if _nvls_kernel_ok(tensor, op) and (nbytes > PUSH_MAX_BYTES or _is_symmetric(tensor)):
                algorithm = "nvls_kernel"
        elif routed[0] is not None and (routed[0] not in ("ll", "push") or
                                        (_ll_eligible if routed[0] == "ll" else _push_eligible)(tensor, op, routed[0])):
            algorithm, channels = routed[0], channels or routed[1]
    if algorithm == "nvls_kernel":
        if not _nvls_kernel_ok(tensor, op):
            raise ValueError("the in-switch all-reduce kernel takes f32/f16/bf16 sums of a multiple of 16 * world "
                             "bytes on an engine with NVLS")
        _nvls_kernel(tensor)
        return tensor
    if _ll_eligible(tensor, op, algorithm):
        ll = _state["ll"]
        ll["epoch"] += 1
        work = _aligned(tensor, 8)
        ll["native"].allreduce_ll(work, work, ll["buf"].heap_offset, LL_MAX_BYTES, ll["epoch"], _state["err_ll"])
        if work is not tensor:
            tensor.copy_(work)
        return tensor
    if _push_eligible(tensor, op, algorithm):
        _push(0, tensor, tensor)
        return tensor
    if algorithm == "push":
        raise ValueError("the push all-reduce takes f32/f16/bf16 sums of a multiple of 16 and at most "
                         f"{PUSH_MAX_BYTES} bytes")
    if algorithm == "ll":
        raise ValueError("the packet-protocol all-reduce takes f32/f16/bf16 sums of a multiple of 8 and at most "
                         f"{LL_MAX_BYTES} bytes")
    name = ensure_plan("allreduce", tensor.numel(), tensor.dtype, algorithm, channels, op)
    run = _engine.execute_operation_async if async_op else _engine.execute_operation
    run(name, tensor, tensor)
    return tensor


def _run(name: str, input: torch.Tensor, output: torch.Tensor, async_op: bool) -> None:
    (_engine.execute_operation_async if async_op else _engine.execute_operation)(name, input, output)


def reduce_scatter(output: torch.Tensor, input: torch.Tensor, op: str = "sum",
                   algorithm: Optional[str] = None, channels: Optional[int] = None,
                   async_op: bool = False) -> torch.Tensor:
    """``async_op``: enqueue on the current stream and return (``synchronize`` checks the status later).

    Sums of up to ``PUSH_MAX_BYTES`` run in the fused push kernel unless an algorithm is forced."""
    if output.numel() * _state["world"] == input.numel():
        if _ll_part_ok(output, input, algorithm, op=op, kind="reduce_scatter"):
            _ll_collective(1, input, output)
            return output
        if _push_ok(input, output, algorithm, op=op):
            _push(1, input, output)
            return output
    if algorithm in ("ll", "push"):
        raise ValueError(f"the {algorithm} reduce-scatter takes f32/f16/bf16 sums within its size limit")
    name = ensure_plan("reduce_scatter", input.numel(), input.dtype, algorithm, channels, op)
    _run(name, input, output, async_op)
    return output


def all_gather(output: torch.Tensor, input: torch.Tensor, algorithm: Optional[str] = None,
               channels: Optional[int] = None, executor: Optional[str] = None,
               async_op: bool = False) -> torch.Tensor:
    """``executor="ce"`` moves the shards with the copy engines (``algorithm`` twoshot)."""
    if input.numel() * _state["world"] == output.numel():
        if _ll_part_ok(input, output, algorithm, executor, kind="allgather"):
            _ll_collective(2, input, output)
            return output
        if _push_ok(output, input, algorithm, executor):
            _push(2, input, output)
            return output
    if algorithm in ("ll", "push"):
        raise ValueError(f"the {algorithm} all-gather takes f32/f16/bf16 tensors within its size limit")
    if executor == "ce":
        algorithm = "twoshot"
    name = ensure_plan("allgather", output.numel(), output.dtype, algorithm, channels, executor=executor)
    _run(name, input, output, async_op)
    return output


def all_to_all(output: torch.Tensor, input: torch.Tensor, algorithm: Optional[str] = None,
               channels: Optional[int] = None, executor: Optional[str] = None,
               async_op: bool = False) -> torch.Tensor:
    if input.numel() == output.numel() and input.numel() % _state["world"] == 0:
        if _ll_part_ok(input[:input.numel() // _state["world"]], output, algorithm, executor):
            _ll_collective(3, input, output)
            return output
        if _push_ok(input, output, algorithm, executor):
            _push(3, input, output)
            return output
    if algorithm in ("ll", "push"):
        raise ValueError(f"the {algorithm} all-to-all takes f32/f16/bf16 tensors within its size limit")
    if executor == "ce":
        algorithm = "twoshot"
    name = ensure_plan("alltoall", input.numel(), input.dtype, algorithm or "twoshot", channels, executor=executor)
    _run(name, input, output, async_op)
    return output


_FUSED_CODES = {0x701: "packet all-reduce: a peer's packets did not arrive",
                0x801: "push collective: a peer's first flag did not arrive",
                0x802: "push collective: a peer's second flag did not arrive",
                0x901: "in-switch all-reduce: a peer's input flag did not arrive",
                0x902: "in-switch all-reduce: a peer's delivery flag did not arrive"}


def check_errors() -> None:
    """Raise ``PCCLTimeoutError`` if a fused collective of this layer gave up waiting since the last check.
    Synchronises the current stream's device (it reads the kernels' error words)."""
    errors = _state.get("errors")
    if errors is None:
        return
    codes = errors.tolist()
    if any(codes):
        what = "; ".join(_FUSED_CODES.get(c, hex(c)) for c in codes if c)
        raise _engine.PCCLTimeoutError(f"rank {_state['rank']}: {what}; call pccl_b200.parallel.reset() on every rank "
                                       "before running collectives again")


def synchronize(name: str = "") -> None:
    """Wait for the current stream and surface device-side timeouts: of plans (the engine's status
    block) and of the fused packet / push kernels (their error words)."""
    _engine.sync_operation(name)
    check_errors()


def reset() -> None:
    """Bring every rank's collective state back to its initial value after an error (a timeout leaves
    call counters, flags and receive buffers out of step between ranks).  Collective: every rank calls
    it; it synchronises the device and the group."""
    group = _state["group"]
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if dist.is_initialized() and _state["world"] > 1:
        dist.barrier(group=group)
    ll, push, errors = _state.get("ll"), _state.get("push"), _state.get("errors")
    if ll is not None:
        ll["buf"].zero_()
        ll["epoch"] = 0
    if push is not None:
        push["flags"].zero_()
        push["counters"].zero_()
        push["epoch"] = 0
    lean = _state.get("push_lean")
    if lean is not None:
        lean["flags"].zero_()
        lean["counters"].zero_()
        lean["epoch"] = 0
    nvls = _state.get("nvls")
    if nvls is not None:
        nvls["flags"].zero_()
        nvls["counter"].zero_()
        nvls["epoch"] = 0
    if errors is not None:
        errors.zero_()
    engine = _engine.get_engine()
    if hasattr(engine, "reset"):
        engine.reset()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if dist.is_initialized() and _state["world"] > 1:
        dist.barrier(group=group)


def registered_plans() -> Dict[str, Tuple[str, str, int]]:
    return dict(_state["registered"])
