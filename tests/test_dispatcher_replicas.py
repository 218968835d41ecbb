"""The dispatcher that dispatches, on the host: worker processes with a stand-in engine (no GPU), one prompt
list in, one merged result list out, and the shares of a worker that dies or raises sent to the others."""
import os
from types import SimpleNamespace

import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

from mini_vllm_b200.config import SamplingParams
from mini_vllm_b200.dispatcher import ReplicatedEngine, WorkerLost, generate_over_ranks
from mini_vllm_b200.workloads import config2_requests


def completion(prompt: list[int], max_tokens: int) -> list[int]:
    """What the stand-in model generates: a function of the request alone."""
    s = sum(prompt) % 100003
    return [(s * 31 + i * 17) % 151936 for i in range(max_tokens)]


class StandInEngine:
    """``generate`` with the Engine's contract.  ``fail`` makes replica ``device`` misbehave on its first job."""

    def __init__(self, config, device: int):
        self.config, self.device, self.jobs = config, device, 0
        if config.fail == ("start", device):
            raise RuntimeError("this replica cannot come up")

    def generate(self, prompts, sampling_params, use_tqdm=False):
        self.jobs += 1
        if self.jobs == 1 and self.config.fail == ("raise", self.device):
            raise RuntimeError("device error on this replica")
        if self.jobs == 1 and self.config.fail == ("exit", self.device):
            os._exit(3)                                # killed between steps: no goodbye, the pipe just closes
        return [{"prompt": None, "completion": None, "tokens": completion(p, sp.max_tokens), "replica": self.device}
                for p, sp in zip(prompts, sampling_params)]


def stand_in_factory(config, device_index):
    return StandInEngine(config, device_index)


def workload(n=48):
    reqs = config2_requests(seed=3, n=n)
    return [r.prompt for r in reqs], [SamplingParams(max_tokens=min(r.max_tokens, 40), ignore_eos=True) for r in reqs]


def test_one_prompt_list_in_one_merged_list_out():
    prompts, params = workload()
    with ReplicatedEngine(SimpleNamespace(fail=None), devices=3, engine_factory=stand_in_factory) as eng:
        assert eng.num_replicas == 3
        out = eng.generate(prompts, params)
        again = eng.generate(prompts[:5], params[0])           # a second job, one SamplingParams for all
    assert [o["tokens"] for o in out] == [completion(p, sp.max_tokens) for p, sp in zip(prompts, params)]
    assert {o["replica"] for o in out} == {0, 1, 2}
    assert [o["tokens"] for o in again] == [completion(p, params[0].max_tokens) for p in prompts[:5]]
    assert not eng.lost and eng.requeued == 0


@pytest.mark.parametrize("how", ["raise", "exit"])
def test_a_lost_replica_has_its_share_requeued(how):
    prompts, params = workload()
    with ReplicatedEngine(SimpleNamespace(fail=(how, 1)), devices=3, engine_factory=stand_in_factory) as eng:
        out = eng.generate(prompts, params)
        assert eng.num_replicas == 2 and [w for w, _ in eng.lost] == [1]
        assert eng.requeued > 0
        assert [o["tokens"] for o in out] == [completion(p, sp.max_tokens) for p, sp in zip(prompts, params)]
        assert {o["replica"] for o in out} == {0, 2}
        out2 = eng.generate(prompts[:7], params[:7])            # the survivors keep serving
        assert [o["tokens"] for o in out2] == [completion(p, sp.max_tokens) for p, sp in zip(prompts[:7], params[:7])]


def test_replicas_that_do_not_start():
    prompts, params = workload(12)
    with ReplicatedEngine(SimpleNamespace(fail=("start", 0)), devices=2, engine_factory=stand_in_factory) as eng:
        assert eng.num_replicas == 1 and "cannot come up" in eng.lost[0][1]
        out = eng.generate(prompts, params)
        assert {o["replica"] for o in out} == {1}
    with pytest.raises(WorkerLost, match="no replica could be started"):
        ReplicatedEngine(SimpleNamespace(fail=("start", 0)), devices=1, engine_factory=stand_in_factory)


def test_every_replica_lost_is_an_error():
    prompts, params = workload(8)
    with ReplicatedEngine(SimpleNamespace(fail=("raise", 0)), devices=1, engine_factory=stand_in_factory) as eng:
        with pytest.raises(WorkerLost, match="every replica is gone"):
            eng.generate(prompts, params)


def _rank_main(rank: int, world: int, port: int, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        engine = StandInEngine(SimpleNamespace(fail=None), rank)
        prompts, params = workload(40) if rank == 0 else (None, None)
        out = generate_over_ranks(engine, prompts, params, group=dist.new_group(backend="gloo"))
        if rank == 0:
            assert [o["tokens"] for o in out] == [completion(p, sp.max_tokens) for p, sp in zip(prompts, params)]
            ret["replicas"] = sorted({o["replica"] for o in out})
        else:
            assert out is None
    finally:
        dist.destroy_process_group()


def test_dispatch_between_two_gloo_ranks():
    world, port = 2, 29741
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_rank_main, args=(world, port, ret), nprocs=world, join=True)
        assert ret["replicas"] == [0, 1]
