"""Host side of the Nupovik family, no GPU: the config reader's expansion of layers + loop into layer runs, its
refusals, the checkpoint checks of load_weights, the pool shapes the model asks for, and the oracle's own
consistency (a sequence fed in portions equals the sequence fed at once)."""
import json

import pytest
import torch

from oracle import nupovik_oracle as N
from tests import nupovik_helpers as C
from tests import rimidra_helpers as H


def _folder(tmp_path, cfg, weights=None):
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    if weights is not None:
        H.write_safetensors(str(tmp_path / "model.safetensors"), weights)
    return str(tmp_path)


@pytest.mark.parametrize("name", list(C.CONFIGS))
def test_layer_runs_follow_the_loop(tmp_path, name):
    from semi_pd_b200.configs import get_model_config
    cfg = C.CONFIGS[name]()
    mc = get_model_config(_folder(tmp_path, cfg))
    runs = N.layer_runs(cfg)
    assert mc.model_type == "nupovik" and mc.num_hidden_layers == len(runs)
    assert [(s["layer"], s["opens_pass"]) for s in mc.layer_specs] == runs
    first = {}
    for r, s in enumerate(mc.layer_specs):
        assert s["weights_of"] == first.get(s["layer"])
        first.setdefault(s["layer"], r)
    assert mc.hidden_size == cfg["width"] and mc.vocab_size == cfg["vocab"]
    assert mc.rms_norm_eps == cfg["norm"]["eps"] and mc.logit_scale == cfg.get("logit_scale", 1.0)


def test_reader_refuses_what_it_does_not_know(tmp_path):
    from semi_pd_b200.configs import get_model_config
    good = C.config_mixed()
    for change in (lambda c: c["layers"][0].update(type="conv"),
                   lambda c: c["layers"][0]["mlp"].update(kind="gated"),
                   lambda c: c["loop"].update(stop=9),
                   lambda c: c["loop"].update(start=2, stop=2),
                   lambda c: c["loop"].update(times=0),
                   lambda c: c.update(architecture="Other")):
        cfg = json.loads(json.dumps(good))
        change(cfg)
        with pytest.raises(ValueError):
            get_model_config(_folder(tmp_path, cfg))


def test_checkpoint_is_checked_against_the_config(tmp_path):
    from semi_pd_b200.configs import get_model_config
    from semi_pd_b200.nupovik import NupovikForCausalLM
    cfg = C.config_mixed()
    w = N.make_weights(cfg, seed=1, low_rank=5)  # the low-rank size is the checkpoint's to choose
    model = NupovikForCausalLM(get_model_config(_folder(tmp_path, cfg)), dtype=torch.float32, device="cpu")
    model.load_weights(w.items())
    kv, st, sh = model.cache_shapes()
    kinds = [cfg["layers"][i]["type"] for i, _ in N.layer_runs(cfg)]
    for r, kind in enumerate(kinds):
        m = cfg["layers"][N.layer_runs(cfg)[r][0]]["mixer"]
        if kind == "latent_attention":
            assert kv[r] == (1, m["kv_rank"], 0) and st[r] is None and sh[r] is None
        else:
            assert kv[r] is None and st[r] == (m["heads"], m["dim"], m.get("vdim", m["dim"]))
            assert sh[r] == (cfg["width"] if kind == "wkv" else None)
    # runs of one layer share tensors, not caches
    assert model.layers[0].mixer.r is model.layers[2].mixer.r and model.layers[0].layer_id != model.layers[2].layer_id
    missing = dict(w)
    del missing["l1.mix.uk"]
    with pytest.raises(KeyError):
        model.load_weights(missing.items())
    wrong = dict(w)
    wrong["l2.mix.norm"] = torch.zeros(7)
    with pytest.raises(ValueError):
        model.load_weights(wrong.items())
    uneven = dict(w)
    uneven["l2.mix.a2"] = torch.zeros(w["l2.mix.a2"].shape[0], 6)
    with pytest.raises(ValueError):
        model.load_weights(uneven.items())


def test_pool_with_a_latent_layer_and_vector_state():
    from semi_pd_b200.memory_pool import HybridTokenToKVPool, RecurrentStatePool
    states = RecurrentStatePool(3, [None, (2, 4, 6)], device="cpu", shift_dims=[None, 10])
    assert states.get_state(1).shape == (3, 2, 4, 6) and states.get_shift(1).shape == (3, 10)
    assert states.get_shift(0) is None
    assert RecurrentStatePool.bytes_per_slot([None, (2, 4, 6)], [None, 10]) == 4 * (48 + 10)
    pool = HybridTokenToKVPool(16, 1, torch.float32, [(1, 12, 0), None, (2, 4, 6)], device="cpu", state_pool=states)
    assert pool.get_value_buffer(0) is pool.get_key_buffer(0) and pool.get_key_buffer(0).shape == (17, 1, 12)
    assert pool.get_key_buffer(1) is None and pool.get_value_buffer(2).shape == (17, 2, 6)
    assert HybridTokenToKVPool.bytes_per_token([(1, 12, 0), None, (2, 4, 6)], torch.float32) == 4 * (12 + 2 * 10)
    k, v = pool.get_kv_size_bytes()
    assert k == 4 * 17 * (12 + 8) and v == 4 * 17 * 12  # the latent buffer is counted once


@pytest.mark.parametrize("name", ["mixed", "ones"])
def test_oracle_in_portions_equals_oracle_at_once(name):
    cfg = C.CONFIGS[name]()
    w = N.make_weights(cfg, seed=C.SEEDS[name], low_rank=4)
    toks = H.prompt(23, cfg["vocab"], 5)
    whole = N.forward(cfg, w, toks)
    st = N.Stepper(cfg, w)
    parts = torch.cat([st.feed(toks[a:b]) for a, b in ((0, 1), (1, 3), (3, 14), (14, 15), (15, 23))])
    assert (parts - whole).abs().max().item() < 1e-9
