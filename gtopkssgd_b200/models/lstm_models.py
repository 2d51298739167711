"""DeepSpeech-style acoustic model for AN4 (reference: models/lstm_models.py:21-287):
two masked 2-D convolutions over the spectrogram, ``nb_layers`` recurrent layers
with sequence-wise batch norm, a lookahead convolution for unidirectional nets,
and a batch-normed linear classifier.  Module names match the reference so its
``state_dict`` / ``serialize`` packages load."""
from __future__ import annotations

import math
from collections import OrderedDict

import torch
import torch.nn as nn
import torch.nn.functional as F

supported_rnns = {"lstm": nn.LSTM, "rnn": nn.RNN, "gru": nn.GRU}
supported_rnns_inv = {v: k for k, v in supported_rnns.items()}


class SequenceWise(nn.Module):
    """Applies a module to (T*N, H) and restores (T, N, H)."""

    def __init__(self, module: nn.Module):
        super().__init__()
        self.module = module

    def forward(self, x):
        t, n = x.shape[:2]
        return self.module(x.reshape(t * n, -1)).view(t, n, -1)


class MaskConv(nn.Module):
    """Runs a conv stack on (B, C, D, T) and zeroes everything past each
    sample's valid length after every layer."""

    def __init__(self, seq_module: nn.Sequential):
        super().__init__()
        self.seq_module = seq_module

    def forward(self, x, lengths):
        lengths = torch.as_tensor(lengths, device=x.device)
        for layer in self.seq_module:
            x = layer(x)
            steps = torch.arange(x.size(3), device=x.device)
            pad = steps.view(1, 1, 1, -1) >= lengths.view(-1, 1, 1, 1)
            x = x.masked_fill(pad, 0)
        return x, lengths


class InferenceBatchSoftmax(nn.Module):
    def forward(self, x):
        return x if self.training else F.softmax(x, dim=-1)


class BatchRNN(nn.Module):
    def __init__(self, input_size, hidden_size, rnn_type=nn.LSTM, bidirectional=False, batch_norm=True):
        super().__init__()
        self.input_size, self.hidden_size, self.bidirectional = input_size, hidden_size, bidirectional
        self.batch_norm = SequenceWise(nn.BatchNorm1d(input_size)) if batch_norm else None
        self.rnn = rnn_type(input_size=input_size, hidden_size=hidden_size, bidirectional=bidirectional, bias=True)
        self.num_directions = 2 if bidirectional else 1

    def flatten_parameters(self):
        self.rnn.flatten_parameters()

    def forward(self, x, output_lengths):
        if self.batch_norm is not None:
            x = self.batch_norm(x)
        total = x.size(0)
        x = nn.utils.rnn.pack_padded_sequence(x, output_lengths.cpu())
        x, _ = self.rnn(x)
        x, _ = nn.utils.rnn.pad_packed_sequence(x, total_length=total)
        if self.bidirectional:
            x = x.view(x.size(0), x.size(1), 2, -1).sum(2)
        return x


class Lookahead(nn.Module):
    """Lookahead convolution (Wang et al. 2016): each step mixes the next
    ``context`` steps per feature.  Input and output are (T, N, H)."""

    def __init__(self, n_features: int, context: int):
        super().__init__()
        assert context > 0
        self.n_features, self.context = n_features, context
        self.weight = nn.Parameter(torch.empty(n_features, context + 1))
        self.register_parameter("bias", None)
        bound = 1.0 / math.sqrt(self.weight.size(1))
        nn.init.uniform_(self.weight, -bound, bound)

    def forward(self, x):
        t = x.size(0)
        x = F.pad(x, (0, 0, 0, 0, 0, self.context))
        windows = x.unfold(0, self.context + 1, 1)[:t]  # (T, N, H, context+1)
        return (windows * self.weight).sum(dim=3)


class DeepSpeech(nn.Module):
    def __init__(self, rnn_type=nn.LSTM, labels="abc", rnn_hidden_size=768, nb_layers=5, audio_conf=None,
                 bidirectional=True, context=20):
        super().__init__()
        self.name = "lstman4"
        self._version = "0.0.1"
        self._hidden_size, self._hidden_layers, self._rnn_type = rnn_hidden_size, nb_layers, rnn_type
        self._audio_conf = audio_conf or {}
        self._labels, self._bidirectional, self._context = labels, bidirectional, context
        sample_rate = self._audio_conf.get("sample_rate", 16000)
        window_size = self._audio_conf.get("window_size", 0.02)
        self.conv = MaskConv(nn.Sequential(
            nn.Conv2d(1, 32, (41, 11), stride=(2, 2), padding=(20, 5)), nn.BatchNorm2d(32),
            nn.Hardtanh(0, 20, inplace=True),
            nn.Conv2d(32, 32, (21, 11), stride=(2, 1), padding=(10, 5)), nn.BatchNorm2d(32),
            nn.Hardtanh(0, 20, inplace=True)))
        feat = int(math.floor(sample_rate * window_size / 2) + 1)
        feat = int(math.floor(feat + 2 * 20 - 41) / 2 + 1)
        feat = int(math.floor(feat + 2 * 10 - 21) / 2 + 1)
        feat *= 32
        layers = [("0", BatchRNN(feat, rnn_hidden_size, rnn_type, bidirectional, batch_norm=False))]
        for i in range(1, nb_layers):
            layers.append((str(i), BatchRNN(rnn_hidden_size, rnn_hidden_size, rnn_type, bidirectional)))
        self.rnns = nn.Sequential(OrderedDict(layers))
        self.lookahead = None if bidirectional else nn.Sequential(Lookahead(rnn_hidden_size, context),
                                                                  nn.Hardtanh(0, 20, inplace=True))
        self.fc = nn.Sequential(SequenceWise(nn.Sequential(nn.BatchNorm1d(rnn_hidden_size),
                                                           nn.Linear(rnn_hidden_size, len(labels), bias=False))))
        self.inference_softmax = InferenceBatchSoftmax()

    def get_seq_lens(self, input_length):
        n = torch.as_tensor(input_length).clone()
        for m in self.conv.modules():
            if isinstance(m, nn.Conv2d):
                n = torch.div(n + 2 * m.padding[1] - m.dilation[1] * (m.kernel_size[1] - 1) - 1, m.stride[1],
                              rounding_mode="floor") + 1
        return n.int()

    def forward(self, x, lengths):
        out_len = self.get_seq_lens(torch.as_tensor(lengths).cpu().int())
        x, _ = self.conv(x, out_len)
        b, c, dfeat, t = x.shape
        x = x.view(b, c * dfeat, t).permute(2, 0, 1).contiguous()  # T x N x H
        for rnn in self.rnns:
            x = rnn(x, out_len)
        if self.lookahead is not None:
            x = self.lookahead(x)
        x = self.fc(x).transpose(0, 1)
        return self.inference_softmax(x), out_len

    # -- (de)serialisation package of the reference (lstm_models.py:240-287) ----
    @staticmethod
    def is_parallel(model):
        return isinstance(model, (nn.DataParallel, nn.parallel.DistributedDataParallel))

    @staticmethod
    def serialize(model, optimizer=None, epoch=None, iteration=None, loss_results=None, cer_results=None,
                  wer_results=None, avg_loss=None, meta=None):
        m = model.module if DeepSpeech.is_parallel(model) else model
        pkg = {"version": m._version, "hidden_size": m._hidden_size, "hidden_layers": m._hidden_layers,
               "rnn_type": supported_rnns_inv.get(m._rnn_type, m._rnn_type.__name__.lower()),
               "audio_conf": m._audio_conf, "labels": m._labels, "state_dict": m.state_dict(),
               "bidirectional": m._bidirectional, "context": m._context}
        if optimizer is not None:
            pkg["optim_dict"] = optimizer.state_dict()
        for key, val in (("avg_loss", avg_loss), ("iteration", iteration), ("meta", meta)):
            if val is not None:
                pkg[key] = val
        if epoch is not None:
            pkg["epoch"] = epoch + 1
        if loss_results is not None:
            pkg.update(loss_results=loss_results, cer_results=cer_results, wer_results=wer_results)
        return pkg

    @classmethod
    def load_model_package(cls, package):
        model = cls(rnn_hidden_size=package["hidden_size"], nb_layers=package["hidden_layers"],
                    labels=package["labels"], audio_conf=package["audio_conf"],
                    rnn_type=supported_rnns[package["rnn_type"]], bidirectional=package.get("bidirectional", True),
                    context=package.get("context", 20))
        model.load_state_dict(package["state_dict"])
        return model

    @classmethod
    def load_model(cls, path):
        model = cls.load_model_package(torch.load(path, map_location="cpu", weights_only=False))
        for r in model.rnns:
            r.flatten_parameters()
        return model

    @staticmethod
    def get_param_size(model):
        return sum(p.numel() for p in model.parameters())

    @staticmethod
    def get_labels(model):
        return (model.module if DeepSpeech.is_parallel(model) else model)._labels

    @staticmethod
    def get_audio_conf(model):
        return (model.module if DeepSpeech.is_parallel(model) else model)._audio_conf

    @staticmethod
    def get_meta(model):
        m = model.module if DeepSpeech.is_parallel(model) else model
        return {"version": m._version, "hidden_size": m._hidden_size, "hidden_layers": m._hidden_layers,
                "rnn_type": supported_rnns_inv[m._rnn_type]}


def describe_saved_model(path: str) -> dict:
    """Metadata of a saved DeepSpeech package (what the reference prints from
    ``python lstm_models.py --model-path ...``, lstm_models.py:324-364)."""
    package = torch.load(path, map_location="cpu", weights_only=False)
    model = DeepSpeech.load_model_package(package)
    info = {"model": model.__class__.__name__, "version": package.get("version"),
            "rnn_type": package["rnn_type"], "rnn_layers": package["hidden_layers"],
            "rnn_size": package["hidden_size"], "bidirectional": package.get("bidirectional", True),
            "classes": len(package["labels"]), "labels": package["labels"],
            "parameters": DeepSpeech.get_param_size(model), "audio_conf": package.get("audio_conf", {})}
    for key in ("epoch", "iteration", "avg_loss"):
        if package.get(key) is not None:
            info[key] = package[key]
    if package.get("loss_results") is not None:
        epochs = package.get("epoch", len(package["loss_results"]))
        info["training"] = [{"epoch": i + 1, "loss": float(package["loss_results"][i]),
                             "wer": float(package["wer_results"][i]), "cer": float(package["cer_results"][i])}
                            for i in range(min(int(epochs), len(package["loss_results"])))]
    return info


def main(argv=None):
    import argparse
    import json
    ap = argparse.ArgumentParser(description="Print the metadata of a saved DeepSpeech model")
    ap.add_argument("--model-path", required=True)
    args = ap.parse_args(argv)
    print(json.dumps(describe_saved_model(args.model_path), indent=1, default=str))


if __name__ == "__main__":
    main()
