"""Two-layer LSTM language model for PTB (reference: models/lstm.py:5-47):
embedding = hidden = 1500, dropout 0.65, untied softmax layer, truncated BPTT
over ``num_steps`` tokens with the hidden state carried across iterations."""
from __future__ import annotations

import torch
import torch.nn as nn


class lstm(nn.Module):  # noqa: N801 - name kept for checkpoint / CLI compatibility
    def __init__(self, vocab_size, embedding_dim=1500, num_steps=35, batch_size=20, num_layers=2, dp_keep_prob=0.35):
        super().__init__()
        self.name = "lstm"
        self.embedding_dim, self.num_steps, self.batch_size = embedding_dim, num_steps, batch_size
        self.vocab_size, self.dp_keep_prob, self.num_layers = vocab_size, dp_keep_prob, num_layers
        self.dropout = nn.Dropout(1 - dp_keep_prob)
        self.word_embeddings = nn.Embedding(vocab_size, embedding_dim)
        self.lstm = nn.LSTM(embedding_dim, embedding_dim, num_layers=num_layers, dropout=1 - dp_keep_prob)
        self.sm_fc = nn.Linear(embedding_dim, vocab_size)
        self.init_weights()

    def init_weights(self, init_range: float = 0.1) -> None:
        nn.init.uniform_(self.word_embeddings.weight, -init_range, init_range)
        nn.init.uniform_(self.sm_fc.weight, -init_range, init_range)
        nn.init.zeros_(self.sm_fc.bias)

    def init_hidden(self):
        w = next(self.parameters())
        shape = (self.num_layers, self.batch_size, self.embedding_dim)
        return (w.new_zeros(shape), w.new_zeros(shape))

    def forward(self, inputs, hidden):
        x = self.dropout(self.word_embeddings(inputs))
        out, hidden = self.lstm(x, hidden)
        logits = self.sm_fc(self.dropout(out).reshape(-1, self.embedding_dim))
        return logits.view(self.num_steps, self.batch_size, self.vocab_size), hidden


def repackage_hidden(h):
    """Detach the carried hidden state from the previous iteration's graph."""
    if isinstance(h, torch.Tensor):
        return h.detach()
    return tuple(repackage_hidden(v) for v in h)
