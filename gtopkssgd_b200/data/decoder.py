"""CTC decoders and error rates for the AN4 speech model
(reference: decoder.py:23-197).

``Decoder.wer / cer`` are edit distances over words / characters computed with
a built-in dynamic programme (no python-Levenshtein needed);
``GreedyDecoder`` is the arg-max decoder with blank and repeat removal;
``BeamCTCDecoder`` is a CTC prefix beam search without a language model,
implemented here so that it needs no external ``ctcdecode`` package.
"""
from __future__ import annotations

import math
from collections import defaultdict
from typing import List, Sequence

import torch


def edit_distance(a: Sequence, b: Sequence) -> int:
    """Levenshtein distance between two sequences."""
    if len(a) < len(b):
        a, b = b, a
    prev = list(range(len(b) + 1))
    for i, x in enumerate(a, start=1):
        cur = [i]
        for j, y in enumerate(b, start=1):
            cur.append(min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (x != y)))
        prev = cur
    return prev[-1]


class Decoder:
    def __init__(self, labels, blank_index=0):
        self.labels = labels
        self.int_to_char = {i: c for i, c in enumerate(labels)}
        self.blank_index = blank_index
        self.space_index = labels.index(" ") if " " in labels else len(labels)

    def wer(self, s1: str, s2: str) -> int:
        """Word-level edit distance of two space-separated sentences."""
        return edit_distance(s1.split(), s2.split())

    def cer(self, s1: str, s2: str) -> int:
        """Character-level edit distance, spaces ignored."""
        return edit_distance(s1.replace(" ", ""), s2.replace(" ", ""))

    def decode(self, probs, sizes=None):
        raise NotImplementedError


class GreedyDecoder(Decoder):
    def process_string(self, sequence, size, remove_repetitions=False):
        chars, offsets = [], []
        blank = self.int_to_char[self.blank_index]
        for i in range(int(size)):
            ch = self.int_to_char[int(sequence[i])]
            if ch == blank:
                continue
            if remove_repetitions and i != 0 and ch == self.int_to_char[int(sequence[i - 1])]:
                continue
            chars.append(" " if (self.space_index < len(self.labels) and ch == self.labels[self.space_index]) else ch)
            offsets.append(i)
        return "".join(chars), torch.tensor(offsets, dtype=torch.int)

    def convert_to_strings(self, sequences, sizes=None, remove_repetitions=False, return_offsets=False):
        strings, offsets = [], []
        for x in range(len(sequences)):
            n = sizes[x] if sizes is not None else len(sequences[x])
            s, o = self.process_string(sequences[x], n, remove_repetitions)
            strings.append([s])
            offsets.append([o])
        return (strings, offsets) if return_offsets else strings

    def decode(self, probs, sizes=None):
        """probs: batch x time x classes.  Returns ([[text]], [[offsets]])."""
        best = torch.argmax(probs, dim=2).cpu()
        return self.convert_to_strings(best, sizes, remove_repetitions=True, return_offsets=True)


class BeamCTCDecoder(Decoder):
    """CTC prefix beam search (no language model)."""

    def __init__(self, labels, lm_path=None, alpha=0, beta=0, cutoff_top_n=40, cutoff_prob=1.0, beam_width=100,
                 num_processes=4, blank_index=0):
        super().__init__(labels, blank_index)
        if lm_path is not None:
            raise NotImplementedError("language-model rescoring is not available")
        self.beam_width, self.cutoff_top_n = beam_width, cutoff_top_n

    def _search(self, logp: torch.Tensor) -> str:
        neg_inf = -math.inf

        def lse(*xs):
            m = max(xs)
            return m if m == neg_inf else m + math.log(sum(math.exp(x - m) for x in xs))

        beams = {(): (0.0, neg_inf)}  # prefix -> (log p ending in blank, log p ending in non-blank)
        for t in range(logp.size(0)):
            nxt = defaultdict(lambda: (neg_inf, neg_inf))
            top = torch.topk(logp[t], min(self.cutoff_top_n, logp.size(1)))
            for prefix, (pb, pnb) in beams.items():
                for lp, c in zip(top.values.tolist(), top.indices.tolist()):
                    if c == self.blank_index:
                        b, nb = nxt[prefix]
                        nxt[prefix] = (lse(b, pb + lp, pnb + lp), nb)
                        continue
                    new = prefix + (c,)
                    b, nb = nxt[new]
                    if prefix and prefix[-1] == c:
                        nxt[new] = (b, lse(nb, pb + lp))
                        b2, nb2 = nxt[prefix]
                        nxt[prefix] = (b2, lse(nb2, pnb + lp))
                    else:
                        nxt[new] = (b, lse(nb, pb + lp, pnb + lp))
            beams = dict(sorted(nxt.items(), key=lambda kv: -lse(*kv[1]))[:self.beam_width])
        best = max(beams.items(), key=lambda kv: lse(*kv[1]))[0]
        return "".join(self.int_to_char[c] for c in best)

    def decode(self, probs, sizes=None):
        probs = probs.detach().cpu().float()
        logp = torch.log(probs.clamp_min(1e-30)) if float(probs.min()) >= 0 else torch.log_softmax(probs, -1)
        out: List[List[str]] = []
        for b in range(logp.size(0)):
            n = int(sizes[b]) if sizes is not None else logp.size(1)
            out.append([self._search(logp[b, :n])])
        return out, None
