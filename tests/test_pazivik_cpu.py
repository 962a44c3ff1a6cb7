"""The Pazivik architecture through the engine's host logic on the CPU (plain PyTorch kernels),
against the plain float64 model: configuration, checkpoint layout, shared cache layers, every way
of cutting requests into steps, and greedy generation through the scheduler."""

import copy

import pytest
import torch

import plain_pazivik
import traces
from conftest import PAZIVIK_TINY
from plain_ops import PlainOps


def cpu_runner(folder, name, num_pages, max_num_seqs=4, max_len=512):
    from llmserve_b200.engine.runner import ModelRunner, load_model

    _, _, model = load_model(folder, "float32", "cpu", PlainOps(), max_len)
    return ModelRunner(model, page_tokens=PAZIVIK_TINY[name]["page_tokens"], num_pages=num_pages,
                       max_model_len=max_len, max_num_seqs=max_num_seqs)


def test_config_round_trip_and_refusals():
    from llmserve_b200.config import ConfigError, architecture_for
    from llmserve_b200.config.pazivik import PazivikConfig

    for name in PAZIVIK_TINY:
        d = PAZIVIK_TINY[name]["config"]
        assert architecture_for(d).name == "Pazivik"
        cfg = PazivikConfig.from_dict(d)
        assert cfg.to_dict() == d and PazivikConfig.from_dict(cfg.to_dict()) == cfg
    d = PAZIVIK_TINY["P1"]["config"]
    cfg = PazivikConfig.from_dict(d)
    assert cfg.layers[1].mixer.kv_from == 0 and cfg.layers[2].mlp is None and cfg.layers[3].mlp.shared_ff == 0

    def broken(change):
        b = copy.deepcopy(d)
        change(b)
        with pytest.raises(ConfigError):
            PazivikConfig.from_dict(b)

    broken(lambda b: b["layers"][0].update(type="conv"))
    broken(lambda b: b["layers"][0]["mixer"].pop("scale"))
    broken(lambda b: b["layers"][0]["mixer"].update(rot={"dims": 8}))
    broken(lambda b: b["layers"][1]["mixer"].update(kv_from=1))  # not an earlier layer
    broken(lambda b: b["layers"][3]["mixer"].update(kv_from=1))  # a layer without a latent of its own
    broken(lambda b: b["layers"][1]["mixer"].update(kv_rank=48))  # another rank than the layer it reads
    broken(lambda b: b["layers"][1]["mlp"]["router"].update(top=6))
    broken(lambda b: b["layers"][0]["mlp"].update(kind="conv"))
    broken(lambda b: b["embedding"]["bigram"].pop("mul_prev"))
    broken(lambda b: b["norm"].pop("eps"))


def test_plan_shares_cache_layers_and_keeps_the_widest_window():
    from llmserve_b200.config.pazivik import PazivikConfig
    from llmserve_b200.models.pazivik import pazivik_plan

    plan = pazivik_plan(PazivikConfig.from_dict(PAZIVIK_TINY["P1"]["config"]))
    assert [(e.layer, e.cache) for e in plan.run_order] == [(0, 0), (1, 0), (2, 1), (3, 1)]
    assert [l.mixer.cache_window for l in plan.layers] == [33, 33, 7, 7]
    assert [l.mixer.window for l in plan.layers] == [20, 33, 7, 7]
    assert plan.layers[2].feed_forward is None and not plan.layers[1].mixer.own_latent
    # a rank beyond the kernels' head sizes: every layer of that rank keeps keys and values of its own
    plan4 = pazivik_plan(PazivikConfig.from_dict(PAZIVIK_TINY["P4"]["config"]))
    assert [(e.layer, e.cache) for e in plan4.run_order] == [(0, 0), (1, 1), (2, 2)]
    assert [l.mixer.materialize for l in plan4.layers] == [True, True, False]
    assert [l.mixer.cache_window for l in plan4.layers] == [12, 30, 9] and plan4.layers[1].mixer.latent_key == 0
    plan2 = pazivik_plan(PazivikConfig.from_dict(PAZIVIK_TINY["P2"]["config"]))
    assert [l.mixer.cache_window for l in plan2.layers] == [9, 0, 9]  # the reader sees further than the writer


def test_checkpoint_errors_are_reported_together(pazivik_dirs, tmp_path):
    from safetensors.torch import load_file, save_file

    from llmserve_b200.engine.runner import load_model
    from llmserve_b200.weights.loader import CheckpointError

    t = load_file(str(pazivik_dirs["P1"] / "model.safetensors"))
    assert "l1.mix.dkv" not in t and "l2.norm2" not in t and "l3.mlp.shared.sg" not in t
    t.pop("l1.mlp.e3.up")
    t["l0.mix.sink"] = t["l0.mix.sink"][:-1].contiguous()
    t["l1.mix.dkv"] = torch.zeros(32, 96, dtype=torch.bfloat16)  # a reader has no down-projection
    (tmp_path / "config.json").write_text((pazivik_dirs["P1"] / "config.json").read_text())
    save_file(t, str(tmp_path / "model.safetensors"))
    with pytest.raises(CheckpointError) as e:
        load_model(tmp_path, "float32", "cpu", PlainOps(), 64)
    assert e.value.missing == ["l1.mlp.e3.up"] and e.value.unexpected == ["l1.mix.dkv"]
    assert [w[0] for w in e.value.wrong_shape] == ["l0.mix.sink"]


def test_cache_layers_one_row_per_token_and_the_previous_token(pazivik_dirs):
    runner = cpu_runner(pazivik_dirs["P1"], "P1", 8)
    a, b = runner.pools.view(0, True), runner.pools.view(1, True)
    assert a.k.data_ptr() == a.v.data_ptr() and a.k.shape[1:] == (1, 16, 32)  # one row is key and value
    assert b.k.shape[1:] == (1, 16, 48)  # a rank of 40, padded to the kernels' multiple of 16
    assert [g.planes for g in runner.pools.kv_groups] == [1, 1]
    prev = runner.pools.view(2, True)  # the embedding's cache layer: the token before the next step's first
    assert prev.k is None and prev.state.dtype == torch.int32 and tuple(prev.state.shape[1:]) == (1,)


LENGTHS = {"P1": [5, 70, 1, 33, 49, 26], "P2": [2, 40, 9, 64, 17], "P3": [3, 150, 18, 77], "P4": [4, 60, 1, 45]}


@pytest.mark.parametrize("name", ["P1", "P2", "P3", "P4"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_every_way_of_cutting_matches_plain(pazivik_dirs, name, mode):
    folder = pazivik_dirs[name]
    reqs = traces.make_requests(LENGTHS[name], PAZIVIK_TINY[name]["config"]["vocab"], seed=5)
    expected = {r: plain_pazivik.model_logits(folder, t) for r, t in reqs.items()}
    pool_tokens = traces.tokens_needed(reqs)
    runner = cpu_runner(folder, name, pool_tokens // PAZIVIK_TINY[name]["page_tokens"])
    got = traces.replay(runner, getattr(traces, mode)(reqs))
    traces.compare(got, expected, atol=2e-4, rtol=2e-5)
    assert runner.manager.usage() == 0.0


def test_a_slot_used_again_starts_with_the_first_token_row(pazivik_dirs):
    """Two requests one after the other in an engine with one state slot: the second's first token
    must take the table's last row, whatever token the first left in the slot."""
    folder = pazivik_dirs["P1"]
    reqs = traces.make_requests([40, 37], 211, seed=8)
    expected = {r: plain_pazivik.model_logits(folder, t) for r, t in reqs.items()}
    runner = cpu_runner(folder, "P1", 4, max_num_seqs=1)
    got = traces.replay(runner, traces.portions(reqs))
    traces.compare(got, expected, atol=2e-4, rtol=2e-5)


def engine(folder, name, **kw):
    from llmserve_b200 import EngineConfig, LLMEngine

    d = dict(model=str(folder), dtype="float32", device="cpu", block_size=PAZIVIK_TINY[name]["page_tokens"],
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


PROMPTS = [[5, 9, 100, 31, 7], list(range(40, 77)), [3] * 33, [100, 2]]


def test_greedy_generation_through_the_engine(pazivik_dirs):
    """The scheduler's own portions and batches, then preemption by recomputation (a preempted
    request starts again from position 0 and so from the first-token row)."""
    from llmserve_b200 import SamplingParams

    folder = pazivik_dirs["P1"]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    want = [plain_pazivik.greedy(folder, p, 6) for p in PROMPTS]
    for kw in ({}, {"max_num_batched_tokens": 8}, {"num_kv_blocks": 5, "max_num_batched_tokens": 16}):
        eng = engine(folder, "P1", **kw)
        assert eng._keeps_running_state
        ids = [eng.add_request(p, sp) for p in PROMPTS]
        done = run_all(eng)
        assert [done[i].outputs[0].token_ids for i in ids] == want, kw
        if "num_kv_blocks" in kw:
            assert eng.scheduler.num_preemptions > 0
        assert eng.manager.usage() == 0.0
