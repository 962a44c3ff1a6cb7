"""The Gubotar architecture through the engine's host logic on the CPU (plain PyTorch kernels),
against the plain float64 model: configuration, checkpoint layout, the cache layer with pages and
states side by side, every way of cutting requests into steps, and greedy generation."""

import copy

import pytest
import torch

import plain_gubotar
import traces
from conftest import GUBOTAR_TINY
from plain_ops import PlainOps


def cpu_runner(folder, name, num_pages, max_num_seqs=4, max_len=512):
    from llmserve_b200.engine.runner import ModelRunner, load_model

    _, _, model = load_model(folder, "float32", "cpu", PlainOps(), max_len)
    return ModelRunner(model, page_tokens=GUBOTAR_TINY[name]["page_tokens"], num_pages=num_pages,
                       max_model_len=max_len, max_num_seqs=max_num_seqs)


def test_config_round_trip_and_refusals():
    from llmserve_b200.config import ConfigError, architecture_for
    from llmserve_b200.config.gubotar import GubotarConfig

    d = GUBOTAR_TINY["G1"]["config"]
    assert architecture_for(d).name == "Gubotar"
    cfg = GubotarConfig.from_dict(d)
    assert cfg.to_dict() == d and GubotarConfig.from_dict(cfg.to_dict()) == cfg
    assert [l.type for l in cfg.layers] == ["retention", "parallel", "retention"]
    assert cfg.layers[1].ff == 0 and cfg.layers[0].retention.rot_dims == 8

    def broken(change):
        b = copy.deepcopy(d)
        change(b)
        with pytest.raises(ConfigError):
            GubotarConfig.from_dict(b)

    broken(lambda b: b["layers"][0].update(type="conv"))
    broken(lambda b: b["layers"][0]["mixer"].pop("decay"))
    broken(lambda b: b["layers"][0]["mixer"].update(decay=[0.5]))
    broken(lambda b: b["layers"][1]["mixer"]["left"].update(vdim=8))
    broken(lambda b: b["layers"][1]["mixer"]["left"].update(bias=True))
    broken(lambda b: b["layers"][0]["mixer"]["rot"].update(dims=18))
    broken(lambda b: b["norm"].pop("eps"))


def test_checkpoint_errors_are_reported_together(gubotar_dirs, tmp_path):
    from safetensors.torch import load_file, save_file

    from llmserve_b200.engine.runner import load_model
    from llmserve_b200.weights.loader import CheckpointError

    t = load_file(str(gubotar_dirs["G1"] / "model.safetensors"))
    t.pop("l1.mix.left.temp")
    t["l0.mix.q"] = t["l0.mix.q"][:-1].contiguous()
    t["l1.norm2"] = torch.zeros(96, dtype=torch.bfloat16)  # the unused norm of a layer without feed-forward
    (tmp_path / "config.json").write_text((gubotar_dirs["G1"] / "config.json").read_text())
    save_file(t, str(tmp_path / "model.safetensors"))
    with pytest.raises(CheckpointError) as e:
        load_model(tmp_path, "float32", "cpu", PlainOps(), 64)
    assert e.value.missing == ["l1.mix.left.temp"] and not e.value.unexpected
    assert [w[0] for w in e.value.wrong_shape] == ["l0.mix.q"]


def test_a_cache_layer_holds_pages_and_states_side_by_side(gubotar_dirs):
    runner = cpu_runner(gubotar_dirs["G1"], "G1", 8)
    view = runner.pools.view(1, True)  # the parallel layer: pages, the linear state, the shifted row
    assert view.k is not None and view.k.shape[1:] == (2, 16, 16)
    assert [tuple(s.shape[1:]) for s in view.states] == [(2, 40, 24), (96,)]
    mixer_view, shift_view = view.part(True, 0, 1), view.part(False, 1, 1)
    assert mixer_view.state is view.states[0] and shift_view.state is view.states[1] and shift_view.k is None
    assert [tuple(s.shape[1:]) for s in runner.pools.view(0, True).states] == [(3, 32, 16), (96,)]
    assert runner.pools.view(0, True).k is None


LENGTHS = {"G1": [5, 70, 1, 33, 49, 26], "G2": [2, 40, 9, 64, 17], "G3": [3, 50, 18, 77], "G4": [5, 70, 33, 100]}


@pytest.mark.parametrize("name", ["G1", "G2", "G3", "G4"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_every_way_of_cutting_matches_plain(gubotar_dirs, name, mode):
    folder = gubotar_dirs[name]
    reqs = traces.make_requests(LENGTHS[name], GUBOTAR_TINY[name]["config"]["vocab"], seed=5)
    expected = {r: plain_gubotar.model_logits(folder, t) for r, t in reqs.items()}
    pool_tokens = traces.tokens_needed(reqs)
    runner = cpu_runner(folder, name, pool_tokens // GUBOTAR_TINY[name]["page_tokens"])
    got = traces.replay(runner, getattr(traces, mode)(reqs))
    traces.compare(got, expected, atol=1e-4)
    assert runner.manager.usage() == 0.0


def test_a_slot_used_again_starts_from_zero(gubotar_dirs):
    """Two requests one after the other in an engine with one state slot: the second must not see
    what the first left in the slot's states."""
    folder = gubotar_dirs["G1"]
    reqs = traces.make_requests([40, 37], 211, seed=8)
    expected = {r: plain_gubotar.model_logits(folder, t) for r, t in reqs.items()}
    runner = cpu_runner(folder, "G1", 4, max_num_seqs=1)
    got = traces.replay(runner, traces.portions(reqs))
    traces.compare(got, expected, atol=1e-4)


def engine(folder, name, **kw):
    from llmserve_b200 import EngineConfig, LLMEngine

    d = dict(model=str(folder), dtype="float32", device="cpu", block_size=GUBOTAR_TINY[name]["page_tokens"],
             num_kv_blocks=64, max_model_len=256, max_num_seqs=8)
    d.update(kw)
    return LLMEngine(EngineConfig(**d), ops=PlainOps())


def run_all(eng):
    done = {}
    while eng.has_unfinished_requests():
        for o in eng.step():
            if o.finished:
                done[o.request_id] = o
        eng.manager.check_invariants()
    return done


PROMPTS = [[5, 9, 100, 31, 7], list(range(40, 57)), [3] * 33, [100, 2]]


def test_greedy_generation_through_the_engine(gubotar_dirs):
    """The scheduler's own portions and batches, then preemption by recomputation (a preempted
    request starts again from position 0, so its states start from zero again)."""
    from llmserve_b200 import SamplingParams

    folder = gubotar_dirs["G1"]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    want = [plain_gubotar.greedy(folder, p, 6) for p in PROMPTS]
    for kw in ({}, {"max_num_batched_tokens": 8}, {"num_kv_blocks": 5, "max_num_batched_tokens": 16}):
        eng = engine(folder, "G1", **kw)
        assert eng._keeps_running_state
        ids = [eng.add_request(p, sp) for p in PROMPTS]
        done = run_all(eng)
        assert [done[i].outputs[0].token_ids for i in ids] == want, kw
        if "num_kv_blocks" in kw:
            assert eng.scheduler.num_preemptions > 0
        assert eng.manager.usage() == 0.0
