"""A stand-in for the step function, for tests of the engine's decisions without a GPU.

Its "model" gives, at the last cached position of a request, the token hash(every token of the request up to that
position) mixed with (seed, index of the generated token): a request's tokens depend on its whole prefix, on its own
sampling parameters and on nothing else, which is what the real step function promises. The runner keeps what
every request has "in the cache" and checks what the engine hands it: positions without gaps, pages reserved for
every position, no page held by two live requests, ids of a step that was queued ahead taken from the step
before it. Ids are computed when a step runs and handed out by `result()`, like the real runner's.

With state slots (`states`, tensors on the CPU) it also plays a mixer with state of its own: a request's slot counts
the tokens the request has run, so a slot that was not zeroed when handed out, is shared by two requests or is
missing shows as a count that differs from where the step starts. `refuse` names prefixes whose row the sampler
refuses (the kernels' answer to a NaN logit): the id is then UNSAMPLABLE.
"""
import zlib

from tiny_inference_engine_b200.cache.manager import blocks_for

VOCAB = 1000
UNSAMPLABLE = -2


def next_token(prefix, seed, index):
    h = zlib.crc32((",".join(map(str, prefix)) + f"|{seed}|{index}").encode())
    return h % VOCAB


def generate_alone(prompt, params, stop=()):
    """What a request generates: the reference for every batching, cutting and preemption."""
    toks, out = list(prompt), []
    for i in range(params.max_tokens):
        t = next_token(toks, params.seed, i)
        toks.append(t)
        out.append(t)
        if t in stop:
            break
    return out


class _Pending:
    def __init__(self, ids, fail):
        self.ids, self.fail = ids, fail

    def result(self):
        if self.fail:
            raise RuntimeError("injected at the read")
        return list(self.ids)


class FakeRunner:
    def __init__(self, cache, max_tokens, max_seqs, states=None):
        self.cache, self.states = cache, states
        self.refuse = lambda prefix: False
        self.max_tokens, self.max_seqs, self.max_logit_rows = max_tokens, max_seqs, max_seqs
        self.cached = {}          # id(request cache) -> tokens whose keys and values it holds
        self.ids = []             # sampled ids of the last step ("on the device")
        self.runs = 0
        self.fail_at = set()      # run numbers that raise before anything is changed
        self.fail_read_at = set() # run numbers whose ids cannot be read (the step itself ran)
        self.synchronized = 0

    def run(self, entries, sampling=None, device_tokens=False):
        self.runs += 1
        if self.runs in self.fail_at:
            raise RuntimeError("injected")
        assert 0 < len(entries) <= self.max_seqs and sum(len(e.tokens) for e in entries) <= self.max_tokens
        page = self.cache.page_size
        owners = {}
        ids, row = [], 0
        for i, e in enumerate(entries):
            assert e.cache.live
            toks = [int(t) for t in e.tokens]
            if device_tokens:
                assert len(toks) == 1
                toks = [self.ids[i]]
            elif getattr(e, "device_row", None) is not None:
                toks[0] = max(self.ids[e.device_row], 0)      # a refused row's id is clamped into the vocabulary
            have = self.cached.setdefault(id(e.cache), [])
            assert e.start <= len(have), f"gap: request holds {len(have)} tokens, step starts at {e.start}"
            del have[e.start:]
            have.extend(toks)
            if self.states is not None and self.states.has_state:
                slot, count = e.cache.state_slot, self.states.tensor(0)
                assert slot >= 0, "a request runs without a state slot"
                assert owners.setdefault(("slot", slot), id(e.cache)) == id(e.cache), "a state slot shared in a step"
                assert int(count[slot, 0]) == e.start, f"state of {int(count[slot, 0])} tokens at position {e.start}"
                count[slot, 0] += len(toks)
            for t in e.cache.tables:
                assert len(t) >= blocks_for(len(have), page), "positions beyond the reserved pages"
                for b in t.held():
                    assert owners.setdefault(b, id(e.cache)) == id(e.cache), "a page held by two requests of a step"
            for w in e.want:
                assert 0 <= w < len(toks)
                if sampling is not None:
                    p, index = sampling[row]
                    prefix = have[:e.start + w + 1]
                    ids.append(UNSAMPLABLE if self.refuse(prefix) else next_token(prefix, p.seed, index))
                row += 1
        if sampling is not None:
            assert len(sampling) == row
        self.ids = ids
        return None, list(ids)

    def fetch(self, logits, ids, sampling):
        return _Pending(ids, self.runs in self.fail_read_at)

    def synchronize(self):
        self.synchronized += 1

    def check(self):
        pass
