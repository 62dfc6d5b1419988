"""CPU: the host side of the Golitar family -- config and registry, the ragged step descriptor, the hybrid cache's slot
and page bookkeeping, the scheduler of HybridEngine.generate (with a stand-in model), the second library's ABI table."""
import json
import os
import re

import pytest
import torch

import golitar_oracle as O
from proxy_inference_engine_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cfg():
    return {"architecture": "Golitar", "vocab": 50, "width": 32, "streams": 2, "norm": {"eps": 1e-5}, "logit_softcap": 9.0,
            "layers": [{"type": "delta", "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "conv": 3}, "mlp": None},
                       {"type": "attention", "mlp": {"kind": "dense", "ff": 40},
                        "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "diff": 0.25, "scale": 0.35,
                                  "mask": {"size": 5}, "rot": {"base": 100.0, "dims": 4}}}]}


def test_hybrid_header_and_binding_table_agree():
    src = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "pie_b200_hybrid.h")).read(), flags=re.S)
    declared = sorted(set(re.findall(r"\b(pieh_[a-z0-9_]+)\s*\(", src)))
    assert declared == sorted(_lib.HYBRID_SIGNATURES)
    L = _lib.load_hybrid(build_if_missing=True)
    for name in declared + ["pie_page_allocator_create", "pie_page_allocate_n"]:
        assert hasattr(L, name)
    assert L.pieh_abi_version() >= 1
    n0 = L.pieh_launch_count()
    assert L.pieh_linear(None, 1, 0, None, 1, 0, None, 1, None, 1, 1, 1, 0, 0.0, None, None, 0, None) == 5   # ENULL
    assert L.pieh_launch_count() == n0


def test_config_and_registry():
    from proxy_inference_engine_b200.checkpoint import MODEL_REGISTRY, model_kind
    from proxy_inference_engine_b200.golitar import GolitarArgs
    a = GolitarArgs.from_dict(_cfg())
    assert (a.vocab, a.width, a.streams, a.norm_eps, a.logit_softcap) == (50, 32, 2, 1e-5, 9.0)
    assert GolitarArgs.from_dict(a.to_dict()).layers == a.layers
    assert model_kind(_cfg()) == "Golitar" and model_kind({"model_type": "llama"}) == "llama"
    assert set(MODEL_REGISTRY) >= {"llama", "Golitar"}
    with pytest.raises(ValueError):
        model_kind({"architecture": "nope"})
    bad = _cfg()
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(ValueError):
        GolitarArgs.from_dict(bad)
    bad = _cfg()
    bad["layers"][1]["mlp"]["kind"] = "experts"
    with pytest.raises(ValueError):
        GolitarArgs.from_dict(bad)


@pytest.mark.parametrize("rot", [{"base": 1e4, "dims": 16},
                                 {"base": 5e5, "dims": 32, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 256}},
                                 {"base": 100.0, "dims": 8, "scaling": {"factor": 2.0, "low": 2.0, "high": 3.0, "original": 40}}])
def test_rotary_frequencies_match_the_restatement(rot):
    from proxy_inference_engine_b200.golitar import scaled_rotary_frequencies
    got = torch.tensor(scaled_rotary_frequencies(rot), dtype=torch.float64)
    assert torch.allclose(got, O.rotary_freqs(rot), rtol=1e-12, atol=0)
    if "scaling" in rot:   # all three branches occur
        plain = torch.tensor(scaled_rotary_frequencies({k: v for k, v in rot.items() if k != "scaling"}), dtype=torch.float64)
        ratio = got / plain
        assert ratio.max() == 1.0 and abs(float(ratio.min()) - 1.0 / rot["scaling"]["factor"]) < 1e-12


def test_random_checkpoint_has_the_design_tensor_names():
    from proxy_inference_engine_b200.golitar import GolitarArgs, random_weights
    w = random_weights(GolitarArgs.from_dict(_cfg()))
    for name in ("embed", "head", "final.norm", "l0.norm1", "l0.mix.q.conv", "l0.mix.A_log", "l0.mix.dt_bias", "l0.hc1.mix",
                 "l1.mix.q.b", "l1.mix.k.norm", "l1.mix.lq2", "l1.mix.o.b", "l1.mlp.up", "l1.hc2.in", "l1.norm2"):
        assert name in w, name
    assert "l0.norm2" not in w and w["l1.mix.q"].shape == (2 * 2 * 8, 32) and w["l0.mix.q.conv"].shape == (8, 3)
    logits = O.forward(_cfg(), w, [1, 2, 3, 4, 5, 6, 7])
    assert logits.shape == (7, 50) and float(logits.abs().max()) <= 9.0


def test_oracle_window_and_recurrence_are_causal():
    """The restatement itself: a token beyond the window or in the future never changes a row."""
    from proxy_inference_engine_b200.golitar import GolitarArgs, random_weights
    cfg = _cfg()
    w = random_weights(GolitarArgs.from_dict(cfg), seed=2)
    ids = list(range(1, 21))
    a = O.forward(cfg, w, ids)
    b = O.forward(cfg, w, ids[:12] + [40] + ids[13:])
    assert torch.equal(a[:12], b[:12]) and not torch.allclose(a[12:], b[12:])


def test_ragged_descriptor_layout():
    from proxy_inference_engine_b200.ragged import BatchDetails
    b = BatchDetails.build([("x", [5, 6, 7], 70, [3, 9], 2), ("y", [8], 0, [4], 0)], device="cpu")
    assert b.state_slots == [2, 0] and b.positions.tolist() == [70, 71, 72, 0]
    d, keep = b.hybrid_descriptor()
    flat = keep[0].tolist()
    assert (d.T, d.n_seq, d.bt_stride) == (4, 2, 2)
    assert flat == [0, 0, 0, 1] + [0, 3] + [3, 1] + [70, 0] + [2, 0] + [0, 1] + [0, 3] and d.n_tiles == 2
    big = BatchDetails.build([("x", list(range(130)), 0, [1, 2, 3], 0), ("y", [1], 5, [4], 1)], device="cpu")
    d2, keep2 = big.hybrid_descriptor()
    assert d2.n_tiles == 4 and keep2[0].tolist()[-8:] == [0, 0, 0, 1, 0, 64, 128, 130]
    assert b.consolidated_block_table.tolist() == [[3, 9], [4, 0]]


def test_hybrid_cache_slots_and_pages_go_round():
    from proxy_inference_engine_b200.cache import HybridCache
    specs = [{"kind": "delta", "H": 2, "dk": 4, "dv": 4, "taps": 3, "channels": 16}, {"kind": "attention", "G": 1, "d": 4, "dv": 4}]
    c = HybridCache(specs, max_tokens=64 * 3, max_seqs=2, device="cpu", lib=_lib.load_hybrid(build_if_missing=True))
    assert c.layers[0]["state"].shape == (2, 2, 4, 4) and c.layers[0]["conv"].shape == (2, 2, 16)
    assert c.layers[1]["k"].shape == (3, 64, 1, 8) and c.layers[1]["v"].dtype == torch.bfloat16
    a, b = c.admit("a"), c.admit("b")
    assert {a["slot"], b["slot"]} == {0, 1}
    with pytest.raises(MemoryError):
        c.admit("c")
    with pytest.raises(ValueError):
        c.admit("a")
    c.reserve("a", 65)
    c.reserve("a", 100)                      # still two pages
    assert len(c.seqs["a"]["pages"]) == 2 and c.can_hold(64, 0) and not c.can_hold(65, 0)
    c.reserve("b", 1)
    with pytest.raises(MemoryError):
        c.reserve("b", 65)
    pages_a, slot_a = list(c.seqs["a"]["pages"]), a["slot"]
    c.release("a")
    n = c.admit("n")
    c.reserve("n", 128)
    assert n["slot"] == slot_a and sorted(n["pages"]) == sorted(pages_a)     # both come back to the next sequence
    c.release("n"); c.release("b")
    assert c.allocator.get_num_free_pages() == 3 and len(c.free_slots) == 2


class _EchoModel:
    """Stands in for a model: logits peak at (last token + 1) mod vocab, so generation counts upwards."""
    device, vocab = "cpu", 11

    def make_cache(self, max_tokens, max_seqs):
        from proxy_inference_engine_b200.cache import HybridCache
        return HybridCache([], max_tokens, max_seqs, device="cpu", lib=_lib.load_hybrid(build_if_missing=True))

    def step(self, batch, cache, rows=None, trace=None):
        self.steps.append((list(batch.sequence_ids), list(batch.input_lengths), list(batch.context_lengths),
                           list(batch.state_slots)))
        out = torch.zeros((rows.numel(), self.vocab))
        for r, row in enumerate(rows.tolist()):
            out[r, (int(batch.token_ids[row]) + 1) % self.vocab] = 1.0
        return out


def test_scheduler_mixes_portions_and_decoding_and_recycles():
    from proxy_inference_engine_b200.engine import HybridEngine
    m = _EchoModel()
    m.steps = []
    eng = HybridEngine(m, max_tokens=64 * 3, max_seqs=2)
    prompts = [[1, 2, 3], list(range(10)) * 7, [4], [9, 9]]          # 3, 70, 1 and 2 tokens
    outs = eng.generate(prompts, max_new_tokens=4, step_tokens=32, sampler=lambda lg: lg.float().argmax(-1))
    assert outs == [[4, 5, 6, 7], [10, 0, 1, 2], [5, 6, 7, 8], [10, 0, 1, 2]]
    assert not eng.cache.seqs and eng.cache.allocator.get_num_free_pages() == 3
    assert all(sum(n) <= 32 for _, n, _, _ in m.steps)
    assert any(len(n) == 2 and 1 in n and max(n) > 1 for _, n, _, _ in m.steps), "a decode row beside a prompt portion"
    assert max(len(ids) for ids, *_ in m.steps) <= 2                     # never more live sequences than slots
    slots = {}
    for ids, _, ctx, sl in m.steps:
        for i, c, s in zip(ids, ctx, sl):
            slots.setdefault(i, set()).add(s)
    assert all(len(s) == 1 for s in slots.values()) and len(slots) == 4   # a sequence keeps its slot; slots are re-used


def test_forward_validates_wanted_rows():
    from proxy_inference_engine_b200.engine import HybridEngine
    m = _EchoModel()
    m.steps = []
    eng = HybridEngine(m, max_tokens=128, max_seqs=1)
    with pytest.raises(ValueError):
        eng.forward([("a", [1, 2], [2])])
    with pytest.raises(ValueError):
        eng.forward([("b", [], None)])
    assert eng.forward([("a", [1, 2], [])]).shape[0] == 0 and eng.cache.seqs["a"]["length"] == 2


def test_trace_runner_refuses_what_a_family_cannot_do(tmp_path):
    from proxy_inference_engine_b200 import trace
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "llama", "quantization": {"group_size": 64, "bits": 4}}))
    assert trace.main(["--model", str(tmp_path), "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"]) == 3
