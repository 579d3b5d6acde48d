"""A stand-in for the model side of the scheduler, for tests without a GPU.

It keeps, like a real cache, what each page slot holds (the token and its position), and its
"logits" at a place are a function of everything the request's block table leads to: a wrong
page, a lost token or a page reused too early changes the next token.
"""
import numpy as np

from sprout_lm_b200.cache import CacheManager, GroupSpec


def next_token(history, vocab):
    acc = 17
    for i, t in enumerate(history):
        acc = (acc * 31 + (i + 1) * (t + 3)) % 1000003
    return acc % vocab


def reference_output(prompt, count, vocab, eos=()):
    out = []
    for _ in range(count):
        token = next_token(list(prompt) + out, vocab)
        out.append(token)
        if token in eos:
            break
    return out


class StubRunner:
    def __init__(self, num_pages, page_tokens, vocab_size=50, max_positions=4096, eos_token_ids=(),
                 prefix_caching=True, state_slots=0):
        self.vocab_size, self.max_positions, self.eos_token_ids = vocab_size, max_positions, tuple(eos_token_ids)
        self.page_tokens = page_tokens
        self.manager = CacheManager([GroupSpec("full", "full", None, (0,))], num_pages, page_tokens,
                                    state_slots=state_slots, prefix_caching=prefix_caching)
        self.slots = {}                       # (page, offset) -> (token, position)
        self.steps = []                       # per step: list of (tokens, wanted)
        self.fail_after = None

    def new_sequence(self, tokens=None):
        return self.manager.reuse_prefix(tokens) if tokens is not None else self.manager.create()

    def reserve(self, seq, upto):
        while seq.capacity() < upto:
            if not self.manager.reserve(seq, min(upto, seq.capacity() + self.page_tokens)):
                return False
        return True

    def release(self, seq):
        self.manager.release(seq)

    def step(self, entries):
        if self.fail_after is not None and len(self.steps) >= self.fail_after:
            raise RuntimeError("model failure")
        self.steps.append([(len(e.tokens), list(e.want)) for e in entries])
        logits = []
        for e in entries:
            assert e.seq.capacity() >= e.seq.length + len(e.tokens), "ran a token without a reserved page"
            for i, token in enumerate(e.tokens):
                pos = e.seq.length + i
                self.slots[(e.seq.blocks[pos // self.page_tokens], pos % self.page_tokens)] = (token, pos)
            for w in e.want:
                upto = e.seq.length + w
                history = []
                for p in range(upto + 1):
                    token, at = self.slots[(e.seq.blocks[p // self.page_tokens], p % self.page_tokens)]
                    assert at == p, "a page holds another position's token"
                    history.append(token)
                row = np.zeros(self.vocab_size, dtype=np.float32)
                row[next_token(history, self.vocab_size)] = 4.0
                row[(next_token(history, self.vocab_size) + 1) % self.vocab_size] = 3.0
                logits.append(row)
        for e in entries:
            e.seq.length += len(e.tokens)
        return logits or None

    def sample(self, logits, temperatures, uniforms):
        out = []
        for row, temperature, u in zip(logits, temperatures, uniforms):
            if temperature <= 0:
                out.append(int(np.argmax(row)))
                continue
            p = np.exp((row - row.max()) / temperature)
            c = np.cumsum(p / p.sum())
            out.append(int(min(np.searchsorted(c, u, side="right"), len(row) - 1)))
        return out

    def step_and_sample(self, entries, temperatures, uniforms):
        logits = self.step(entries)
        return self.sample(logits, temperatures, uniforms) if logits else []

    def check_status(self):
        pass
