"""Layers built alike are issued by one call: which layers count as alike, and how the calls of a recorded
layer are turned into a list with (slot, offset) in place of the layer's own addresses. No GPU: models and
caches are built on the CPU and nothing is launched (tests/test_layer_replay_gpu.py compares results)."""
import json

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from tiny_inference_engine_b200 import load_model, make_cache
from tiny_inference_engine_b200.errors import InvalidArgument
from tiny_inference_engine_b200.ops import library, replay
from tiny_inference_engine_b200.parts.layer_runs import LayerRuns, walk_part


@pytest.fixture(autouse=True)
def short_runs(monkeypatch):
    """The tiny model has three layers: let three be a run."""
    monkeypatch.setattr(LayerRuns, "MIN_RUN", 3)


def _model(tmp_path, dtype="bfloat16", **changes):
    cfg = dict(plain.TINY_B, **changes)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    model = load_model(tmp_path, dtype, device="cpu", random_weights=True, seed=0)
    cache, states = make_cache(model, page_size=8, num_pages=12, device="cpu")
    return model, cache, states


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_all_layers_of_the_model_form_one_run(tmp_path, dtype):
    model, cache, states = _model(tmp_path, dtype, num_hidden_layers=5)
    runs = LayerRuns(model, cache, states)
    assert runs.run_end == {0: 4}
    table = runs.table[0]
    assert table.shape[0] == 5 and table.dtype == np.int64 and table.flags.c_contiguous
    # every slot is another tensor in every layer, and the last two slots are the layer's cache planes
    assert len({int(v) for v in table[:, 0]}) == 5
    for i in range(5):
        view = cache.layer_cache(i, writes=True)
        assert (int(table[i, -2]), int(table[i, -1])) == (view.k.data_ptr(), view.v.data_ptr())


def test_two_layers_are_no_run_and_a_moved_tensor_is_noticed(tmp_path):
    model, cache, states = _model(tmp_path, num_hidden_layers=2)
    assert LayerRuns(model, cache, states).run_end == {}
    model, cache, states = _model(tmp_path, num_hidden_layers=3)
    assert LayerRuns(model, cache, states).run_end == {0: 2}
    LayerRuns.MIN_RUN = 4                   # the default: a run shorter than four layers is not worth a list
    assert LayerRuns(model, cache, states).run_end == {}
    LayerRuns.MIN_RUN = 3
    model, cache, states = _model(tmp_path, num_hidden_layers=4)
    runs = LayerRuns(model, cache, states)
    assert runs.run_end == {0: 3} and runs.spans(1, 0) is not None
    assert runs.alive()
    model.layers[1].ffn.w_down = model.layers[1].ffn.w_down.clone()
    assert runs.spans(1, 0) is None
    model.layers[3].ffn.down.w = model.layers[3].ffn.w_down = model.layers[3].ffn.w_down.clone()   # not the recorded layer
    assert not runs.alive()                                 # the old tensor is gone: the model builds the tables anew
    fresh = LayerRuns(model, cache, states)
    moved = model.layers[3].ffn.w_down.data_ptr()
    assert fresh.alive() and moved in fresh.table[0][3].tolist() and moved not in runs.table[0][3].tolist()


def test_the_model_hands_out_runs_after_its_first_forward_and_builds_them_anew_when_a_tensor_is_gone(tmp_path):
    class Ctx:
        layer_hook = None

    model, cache, states = _model(tmp_path, num_hidden_layers=5)
    assert model._runs_for(Ctx(), cache, states) is None          # tensors that parts make at first use may not exist yet
    model._forwards = 1
    runs = model._runs_for(Ctx(), cache, states)
    assert runs is not None and runs.run_end == {0: 4} and model._runs_for(Ctx(), cache, states) is runs
    other_cache, other_states = make_cache(model, page_size=8, num_pages=12, device="cpu")
    assert model._runs_for(Ctx(), other_cache, other_states) is not runs       # tables are per cache: the planes differ
    model.layers[2].mixer_norm.weight = model.layers[2].mixer_norm.weight.clone()
    again = model._runs_for(Ctx(), cache, states)
    assert again is not runs and again.alive() and not runs.alive()
    hooked = Ctx()
    hooked.layer_hook = lambda *a: None
    assert model._runs_for(hooked, cache, states) is None          # a hook wants every layer issued from Python
    model.layer_replay = False
    assert model._runs_for(Ctx(), cache, states) is None


def test_a_layer_that_differs_in_a_constant_or_in_a_part_ends_the_run(tmp_path):
    model, cache, states = _model(tmp_path, num_hidden_layers=7)
    model.layers[3].mixer.scale *= 2.0                      # a constant that is no tensor
    assert LayerRuns(model, cache, states).run_end == {0: 2, 4: 6}
    model.layers[3].mixer.scale /= 2.0
    assert LayerRuns(model, cache, states).run_end == {0: 6}

    class Stranger(type(model.layers[5].ffn)):               # a part that does not promise to launch only
        launches_only = False
    model.layers[5].ffn.__class__ = Stranger
    assert LayerRuns(model, cache, states).run_end == {0: 4}


def test_a_plan_names_the_layers_own_tensors_by_slot_and_offset(tmp_path):
    model, cache, states = _model(tmp_path, num_hidden_layers=4)
    runs = LayerRuns(model, cache, states)
    layer = model.layers[1]
    spans = runs.spans(1, 0)
    tensors, _ = [], []
    walk_part(layer, tensors, _, set())
    shared = 0x7F00_0000_1000                                 # an address outside the layer: stays as it is
    w_k = layer.mixer.w_k.data_ptr()                          # a view into the stacked q/k/v weight
    calls = [("tie_silu_mul", (1, w_k, shared, 7, 200, None)),
             ("tie_rmsnorm_rows", (0, shared, 96, layer.ffn_norm.weight.data_ptr(), 1e-5, shared + 64, 96, 96, 7, 0))]
    p = replay.plan(calls, spans)
    assert p.calls == 2 and list(p.arg_begin) == [0, 6, 16]
    slot_of = {t.data_ptr(): i for i, t in reversed(list(enumerate(tensors)))}      # first tensor at an address
    qkv = slot_of[layer.mixer.w_qkv.data_ptr()]
    assert p.slot[1] == qkv and p.offset[1] == w_k - layer.mixer.w_qkv.data_ptr()
    assert p.slot[9] == slot_of[layer.ffn_norm.weight.data_ptr()] and p.offset[9] == 0
    assert [i for i, s in enumerate(p.slot) if s >= 0] == [1, 9]
    assert p.words[2] == shared and p.words[5] == 0 and p.words[3] == 7
    assert np.int64(p.words[10]).view(np.float64) == 1e-5       # floats travel as the bits of a double
    # the same addresses in another layer's row of the table
    row = runs.table[0][2]
    assert int(row[p.slot[1]]) + int(p.offset[1]) == model.layers[2].mixer.w_k.data_ptr()
    # which arguments are pointers is the launcher's own declaration, not a guess from their size: a 64-bit stride
    # that happens to equal a tensor's address stays a number
    p2 = replay.plan([("tie_rmsnorm_rows", (0, shared, w_k, layer.ffn_norm.weight.data_ptr(), 1e-5, shared, 96, 96, 7, 0))], spans)
    assert p2.slot[2] == -1 and p2.words[2] == w_k and p2.slot[3] >= 0
    # a function that is no launcher of a layer, or a wrong number of arguments: no plan
    assert replay.plan([("tie_sample", (0,) * 9)], spans) is None
    assert replay.plan([("tie_silu_mul", (1, 2, 3))], spans) is None


def test_the_library_checks_a_list_before_it_launches_anything():
    lib = library.library()
    fid = lib.tie_replay_launcher_id(b"tie_silu_mul")
    assert fid >= 0 and lib.tie_replay_launcher_args(fid) == 6 and lib.tie_replay_launcher_id(b"tie_sample") == -1
    good = replay.ReplayPlan(np.array([fid], np.int32), np.array([0, 6], np.int32), np.zeros(6, np.int64),
                             np.full(6, -1, np.int32), np.zeros(6, np.int64), 1, ())
    replay.run(good, np.zeros((0, 3), np.int64))               # no layers: nothing to do
    for bad in (replay.ReplayPlan(good.fn, np.array([0, 5], np.int32), good.words, good.slot, good.offset, 1, ()),
                replay.ReplayPlan(np.array([999], np.int32), good.arg_begin, good.words, good.slot, good.offset, 1, ()),
                replay.ReplayPlan(good.fn, good.arg_begin, good.words, np.full(6, 3, np.int32), good.offset, 1, ())):
        with pytest.raises(InvalidArgument, match="layer replay"):
            replay.run(bad, np.zeros((2, 3), np.int64))
