"""Host dispatcher for multi-GPU serving: independent engine replicas, no tensor crosses GPUs.

The ragged attention path shards only as whole requests, so scaling out means one engine process per GPU
and a host-side split of the request list.  Three layers, lowest first:

* ``partition_by_tokens`` / ``merge_outputs``: the split (longest-first greedy by token cost) and its inverse;
* ``ReplicatedEngine``: the ``Engine.generate`` surface (``minivllm/engine/engine.py:40-90``) in front of one
  worker process per GPU.  The front process partitions a prompt list, sends every worker its share, collects
  the completions and puts them back in submission order.  A worker that exits or raises loses nothing: the
  shares it had not answered are re-partitioned over the workers that are left (the nearest reference
  behaviour is the scheduler re-queueing a preempted request, ``scheduler/scheduler.py:91-98``);
* ``generate_over_ranks``: the same dispatch for processes that already exist as ``torch.distributed`` ranks
  (a ``torchrun`` launch): rank 0 holds the prompts, scatters the shares, every rank runs its own engine,
  rank 0 gathers and merges.  Host objects travel over a gloo group; NCCL is not involved.

Nothing here touches a GPU: the workers own the devices.
"""
from __future__ import annotations

import multiprocessing as mp
import os
import traceback
from multiprocessing.connection import wait as wait_for_connections
from typing import Callable, Sequence


def partition_by_tokens(costs: Sequence[int], n_parts: int) -> list[list[int]]:
    """Longest-first greedy: each request goes to the replica with the fewest tokens so far.

    Returns, per replica, the indices of its requests in ascending (submission) order.  Deterministic:
    ties go to the lower replica index and equal costs keep submission order.
    """
    if n_parts <= 0:
        raise ValueError("n_parts must be positive")
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    loads, parts = [0] * n_parts, [[] for _ in range(n_parts)]
    for i in order:
        j = min(range(n_parts), key=lambda r: (loads[r], r))
        parts[j].append(i)
        loads[j] += costs[i]
    return [sorted(p) for p in parts]


def merge_outputs(parts: list[list[int]], outputs_per_part: list[list], total: int) -> list:
    """Inverse of the partition: ``outputs_per_part[r][k]`` belongs to request ``parts[r][k]``."""
    merged = [None] * total
    for idx, outs in zip(parts, outputs_per_part):
        if len(idx) != len(outs):
            raise ValueError("a replica returned a different number of results than it was given requests")
        for i, o in zip(idx, outs):
            merged[i] = o
    if any(m is None for m in merged):
        raise ValueError("some requests have no result")
    return merged


def request_cost(prompt_len: int, max_tokens: int) -> int:
    """K/V tokens a request reads over its life, one context per generated token: what a replica's time is
    made of.  (Prompt + output alone balances token totals but leaves the attention work uneven.)"""
    return max_tokens * (2 * prompt_len + max_tokens) // 2


def _as_list(sampling_params, n: int) -> list:
    return list(sampling_params) if isinstance(sampling_params, (list, tuple)) else [sampling_params] * n


# ---- worker side -------------------------------------------------------------------------------------------
def default_engine_factory(config, device_index: int):
    """One ``Engine`` on ``cuda:device_index`` (imported here: the front process never needs CUDA)."""
    import torch
    from .engine.engine import Engine
    torch.cuda.set_device(device_index)
    return Engine(config)


def _worker_main(conn, factory: Callable, config, device_index: int) -> None:
    try:
        engine = factory(config, device_index)
        conn.send(("ready", device_index))
        while True:
            msg = conn.recv()
            if msg[0] == "stop":
                break
            _, job_id, prompts, params = msg
            try:
                outs = engine.generate(prompts, params, use_tqdm=False)
                conn.send(("done", job_id, outs))
            except Exception:                         # the engine's state is unknown after a failed job: retire
                conn.send(("failed", job_id, traceback.format_exc()))
                break
    except (EOFError, KeyboardInterrupt):
        pass
    except Exception:
        try:
            conn.send(("failed", None, traceback.format_exc()))
        except Exception:
            pass
    finally:
        conn.close()


class WorkerLost(RuntimeError):
    pass


class ReplicatedEngine:
    """``generate(prompts, sampling_params)`` over one engine replica per device.

    ``devices``: GPU indices (or a count).  ``engine_factory(config, device_index)`` builds what runs in a worker;
    it must be picklable (a module-level function) because workers are spawned, not forked: a forked child
    would inherit a CUDA context it cannot use.
    """

    def __init__(self, config, devices: Sequence[int] | int, engine_factory: Callable | None = None,
                 start_timeout_s: float = 600.0):
        self.config = config
        self.devices = list(range(devices)) if isinstance(devices, int) else list(devices)
        if not self.devices:
            raise ValueError("at least one device is needed")
        ctx = mp.get_context("spawn")
        factory = engine_factory or default_engine_factory
        self._workers: dict[int, tuple] = {}          # worker id -> (process, connection)
        for wid, dev in enumerate(self.devices):
            parent, child = ctx.Pipe()
            proc = ctx.Process(target=_worker_main, args=(child, factory, config, dev), daemon=True)
            proc.start()
            child.close()
            self._workers[wid] = (proc, parent)
        self.lost: list[tuple[int, str]] = []         # (worker id, why) of every worker that went away
        self.requeued = 0                             # requests that had to be sent a second time
        for wid in list(self._workers):
            proc, conn = self._workers[wid]
            try:
                if not conn.poll(start_timeout_s):
                    raise WorkerLost("no answer while starting")
                msg = conn.recv()
                if msg[0] != "ready":
                    raise WorkerLost(str(msg[2]) if len(msg) > 2 else "failed while starting")
            except (EOFError, OSError, WorkerLost) as e:
                self._drop(wid, f"did not start: {e}")
        if not self._workers:
            raise WorkerLost("no replica could be started: " + "; ".join(w for _, w in self.lost))

    # ---- bookkeeping ------------------------------------------------------------------------------------
    @property
    def num_replicas(self) -> int:
        return len(self._workers)

    def _drop(self, wid: int, why: str) -> None:
        proc, conn = self._workers.pop(wid)
        self.lost.append((wid, why))
        try:
            conn.close()
        except OSError:
            pass
        if proc.is_alive():
            proc.terminate()
        proc.join(timeout=5)

    def close(self) -> None:
        for wid in list(self._workers):
            proc, conn = self._workers.pop(wid)
            try:
                conn.send(("stop",))
                conn.close()
            except (OSError, BrokenPipeError):
                pass
            proc.join(timeout=10)
            if proc.is_alive():
                proc.terminate()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False

    # ---- the surface -------------------------------------------------------------------------------------
    def generate(self, prompts: list[list[int]], sampling_params, use_tqdm: bool = False) -> list[dict]:
        """Same contract as ``Engine.generate``: one dict per prompt, in submission order."""
        n = len(prompts)
        params = _as_list(sampling_params, n)
        results: list = [None] * n
        jobs: dict[int, tuple[int, list[int]]] = {}   # job id -> (worker id, request indices)
        next_job = 0

        def send(indices: list[int]) -> None:
            """Partition ``indices`` over the live workers and send each its share."""
            nonlocal next_job
            todo = indices
            while todo:
                if not self._workers:
                    raise WorkerLost("every replica is gone; lost: " + "; ".join(f"{w}: {y}" for w, y in self.lost))
                live = sorted(self._workers)
                costs = [request_cost(len(prompts[i]), params[i].max_tokens) for i in todo]
                shares = partition_by_tokens(costs, len(live))
                again: list[int] = []
                for wid, share in zip(live, shares):
                    if not share:
                        continue
                    idx = [todo[k] for k in share]
                    try:
                        self._workers[wid][1].send(("generate", next_job, [prompts[i] for i in idx],
                                                    [params[i] for i in idx]))
                        jobs[next_job] = (wid, idx)
                        next_job += 1
                    except (OSError, BrokenPipeError) as e:
                        self._drop(wid, f"pipe closed while sending: {e}")
                        again += idx
                todo = again

        def requeue_jobs_of(wid: int) -> None:
            orphaned = [i for j, (w, idx) in list(jobs.items()) if w == wid for i in idx]
            for j in [j for j, (w, _) in jobs.items() if w == wid]:
                del jobs[j]
            self.requeued += len(orphaned)
            send(sorted(orphaned))

        send(list(range(n)))
        while jobs:
            by_conn = {self._workers[w][1]: w for w in {w for w, _ in jobs.values()}}
            by_sentinel = {self._workers[w][0].sentinel: w for w in by_conn.values()}
            ready = wait_for_connections(list(by_conn) + list(by_sentinel))
            seen: set[int] = set()
            for obj in ready:
                wid = by_conn.get(obj, by_sentinel.get(obj))
                if wid in seen or wid not in self._workers:
                    continue
                seen.add(wid)
                proc, conn = self._workers[wid]
                try:
                    if conn.poll():
                        msg = conn.recv()
                    elif not proc.is_alive():
                        raise EOFError(f"process exited with code {proc.exitcode}")
                    else:
                        continue
                except (EOFError, OSError) as e:
                    self._drop(wid, f"went away: {e}")
                    requeue_jobs_of(wid)
                    continue
                if msg[0] == "done":
                    _, job_id, outs = msg
                    w, idx = jobs.pop(job_id)
                    if len(outs) != len(idx):
                        raise ValueError("a replica returned a different number of results than it was given requests")
                    for i, o in zip(idx, outs):
                        results[i] = o
                else:                                  # "failed": the worker retires, its work goes to the others
                    self._drop(wid, "raised:\n" + str(msg[2]))
                    requeue_jobs_of(wid)
        if any(r is None for r in results):
            raise ValueError("some requests have no result")
        return results


# ---- the same dispatch between torch.distributed ranks ---------------------------------------------------------
def generate_over_ranks(engine, prompts, sampling_params, group=None, src: int = 0):
    """Collective: every rank of ``group`` calls this with its own ``engine``; only ``src`` needs ``prompts`` and
    ``sampling_params`` (the others may pass ``None``).  ``src`` partitions the requests by token cost, scatters
    the shares, every rank generates its share, ``src`` gathers the completions and returns them in submission
    order; the other ranks return ``None``.  ``group`` should be a gloo group: the payload is host objects.
    """
    import numpy as np
    import torch.distributed as dist
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    shares = parts = None
    if rank == src:
        params = _as_list(sampling_params, len(prompts))
        parts = partition_by_tokens([request_cost(len(p), sp.max_tokens) for p, sp in zip(prompts, params)], world)
        # token ids travel as one int32 array per share (a pickled list of Python ints is five times the bytes)
        shares = [(np.fromiter((t for i in idx for t in prompts[i]), np.int32),
                   np.fromiter((len(prompts[i]) for i in idx), np.int64, len(idx)), [params[i] for i in idx])
                  for idx in parts]
    mine = [None]
    dist.scatter_object_list(mine, shares, src=dist.get_global_rank(group, src) if group is not None else src,
                             group=group)
    flat, lens, my_params = mine[0]
    cuts = np.concatenate([[0], np.cumsum(lens)])
    my_prompts = [flat[a:b].tolist() for a, b in zip(cuts[:-1], cuts[1:])]
    outs = engine.generate(my_prompts, my_params, use_tqdm=False) if my_prompts else []
    packed = (np.fromiter((t for o in outs for t in o["tokens"]), np.int32),
              np.fromiter((len(o["tokens"]) for o in outs), np.int64, len(outs)),
              [{k: v for k, v in o.items() if k != "tokens"} for o in outs])
    gathered = [None] * world if rank == src else None
    dist.gather_object(packed, gathered, dst=dist.get_global_rank(group, src) if group is not None else src,
                       group=group)
    if rank != src:
        return None
    per_part = []
    for flat, lens, rest in gathered:
        cuts = np.concatenate([[0], np.cumsum(lens)])
        per_part.append([dict(r, tokens=flat[a:b].tolist()) for r, a, b in zip(rest, cuts[:-1], cuts[1:])])
    return merge_outputs(parts, per_part, len(prompts))


def visible_device_count() -> int:
    """GPUs this process may hand to replicas (``CUDA_VISIBLE_DEVICES`` is honoured by the workers' runtime)."""
    env = os.environ.get("CUDA_VISIBLE_DEVICES")
    if env is not None:
        return len([d for d in env.split(",") if d.strip()])
    import torch
    return torch.cuda.device_count()
