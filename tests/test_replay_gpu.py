"""Trace replay through bin/trace_run: the same requests whole, with the last 32 tokens decoded one
by one, in portions of changing size, and mixed with other requests on a pool so small that
pages are used again; float32 and bfloat16; every wanted row against the plain implementation."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_qwen3 as plain
from conftest import ROOT, assert_logits_close

pytestmark = pytest.mark.gpu


class Replay:
    """Drives one trace_run process: a step goes in only after `done` came back for the one before."""

    def __init__(self, model_dir, dtype, out_dir, max_tokens, page_size):
        self.out = Path(out_dir)
        self.proc = subprocess.Popen(
            [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype, "--out",
             str(out_dir), "--max-tokens", str(max_tokens), "--page-size", str(page_size)],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
        self.n = 0

    def step(self, entries, end=()):
        """entries: [(id, tokens, want)]. Returns the logits [wanted, vocab] or None."""
        rec = {"step": self.n, "entries": [{"id": i, "tokens": [int(t) for t in toks], "want": list(w)} for i, toks, w in entries],
               "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        assert line.strip() == f"done {self.n}", f"trace_run answered {line!r}"
        path = self.out / f"{self.n}.f32"
        self.n += 1
        if not any(w for _, _, w in entries):
            assert not path.exists()
            return None
        return np.fromfile(path, dtype="<f4")

    def close(self):
        self.proc.stdin.close()
        assert self.proc.wait(timeout=60) == 0


def cuts_of(n, sizes):
    out, i = [], 0
    while n > 0:
        c = min(n, sizes[i % len(sizes)])
        out.append(c)
        n -= c
        i += 1
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c", "tiny_d", "tiny_e", "tiny_b4"])
def test_replay(tiny_models, tmp_path, name, dtype):
    cfg, page, w, model_dir = tiny_models[name]
    V = cfg["vocab_size"]
    rng = np.random.default_rng(11)
    lengths = [100, 70, 45, 33, 90, 64, 121, 2]
    reqs = [rng.integers(0, V, n).tolist() for n in lengths]
    wq = {k: (plain.round_bf16(v) if v.ndim == 2 else v) for k, v in w.items()} if dtype == "bfloat16" else w
    truth = [plain.forward(wq, cfg, r) for r in reqs]

    # Four live requests of at most 121 tokens, each rounded up to a multiple of 64: 4 * 128.
    rp = Replay(model_dir, dtype, tmp_path, max_tokens=512, page_size=page)
    try:
        # 1. each request alone and whole
        for i, r in enumerate(reqs):
            got = rp.step([(f"w{i}", r, range(len(r)))], end=[f"w{i}"]).reshape(len(r), V)
            assert_logits_close(got, truth[i], dtype, f"{name} whole request {i}")
        # 2. most of it in one step, the last 32 tokens one by one
        for i in (0, 4, 6):
            r, n = reqs[i], len(reqs[i])
            head = n - 32
            got = [rp.step([(f"d{i}", r[:head], range(head))]).reshape(head, V)]
            for t in range(head, n):
                got.append(rp.step([(f"d{i}", r[t:t + 1], [0])], end=[f"d{i}"] if t == n - 1 else []).reshape(1, V))
            assert_logits_close(np.concatenate(got), truth[i], dtype, f"{name} request {i}, last 32 decoded")
        # 3. portions of changing size, down to two tokens
        for i, sizes in ((0, [13, 2, 7, 3, 2, 31]), (1, [2, 2, 5, 17]), (6, [40, 2, 9, 1, 16])):
            r, at, got = reqs[i], 0, []
            cuts = cuts_of(len(r), sizes)
            for j, n in enumerate(cuts):
                got.append(rp.step([(f"c{i}", r[at:at + n], range(n))], end=[f"c{i}"] if j == len(cuts) - 1 else []).reshape(n, V))
                at += n
            assert_logits_close(np.concatenate(got), truth[i], dtype, f"{name} request {i} in portions {sizes}")
        # 4. mixed: up to four live, portions of some beside decoded tokens of others, a request
        #    left out of a step now and then; the pool was filled by the runs above, so every
        #    page handed out here has been used before
        order = [6, 0, 4, 1, 2, 7, 3, 5]
        waiting, live, got = list(order), {}, {i: [] for i in order}
        mix = np.random.default_rng(5)
        steps = 0
        while waiting or live:
            while waiting and len(live) < 4:
                live[waiting.pop(0)] = 0
            entries, ended, owners = [], [], []
            for i, at in list(live.items()):
                left = len(reqs[i]) - at
                if len(live) > 1 and mix.random() < 0.2:
                    continue                       # sits this step out
                n = 1 if left <= 12 else int(min(left - 12, mix.integers(2, 24)))
                want = list(range(n)) if mix.random() < 0.8 else []
                entries.append((f"m{i}", reqs[i][at:at + n], want))
                owners.append((i, at, n, want))
                live[i] = at + n
                if live[i] == len(reqs[i]):
                    ended.append(f"m{i}")
                    del live[i]
            if not entries:
                continue
            out = rp.step(entries, end=ended)
            steps += 1
            if out is None:
                continue
            out = out.reshape(-1, V)
            row = 0
            for i, at, n, want in owners:
                for k in want:
                    got[i].append((at + k, out[row]))
                    row += 1
            assert row == out.shape[0]
        assert steps > 20
        for i in order:
            assert got[i], f"request {i} was never compared"
            pos = [p for p, _ in got[i]]
            assert_logits_close(np.stack([g for _, g in got[i]]), truth[i][pos], dtype, f"{name} request {i} in the mixed run")
    finally:
        rp.close()


def test_pool_too_small_is_an_error_not_a_wrong_answer(tiny_models, tmp_path):
    cfg, page, w, model_dir = tiny_models["tiny_a"]
    rp = Replay(model_dir, "float32", tmp_path, max_tokens=64, page_size=page)
    rec = {"step": 0, "entries": [{"id": "a", "tokens": [1] * 65, "want": [0]}], "end": []}
    rp.proc.stdin.write(json.dumps(rec) + "\n")
    rp.proc.stdin.close()
    assert rp.proc.wait(timeout=120) == 1
