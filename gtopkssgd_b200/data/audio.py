"""Speech data pipeline for AN4 / LibriSpeech-style manifests
(reference: audio_data/data_loader.py:21-318, audio_data/utils.py).

A manifest is a CSV of ``wav path,transcript path`` lines sorted by duration.
``SpectrogramDataset`` turns each utterance into a normalised log-magnitude
STFT (20 ms Hamming window, 10 ms stride -> 161 bins at 16 kHz) and its
transcript into label ids; ``BucketingSampler`` batches neighbours in that
order so padding stays small; ``collate_spectrograms`` pads to the longest
utterance and returns ``(inputs, flat targets, length fractions, target sizes)``.

Only numpy / scipy / torch are required.  Augmentation (speed in [0.85, 1.15],
gain in [-6, 8] dB) and noise injection are done in-process instead of through
the ``sox`` command line.
"""
from __future__ import annotations

import math
import os
import wave
from typing import List, Optional

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset, Sampler

_WINDOWS = {"hamming": torch.hamming_window, "hann": torch.hann_window, "blackman": torch.blackman_window,
            "bartlett": torch.bartlett_window}


def load_audio(path: str) -> np.ndarray:
    """Mono float32 samples in [-1, 1] from a PCM wav file."""
    from scipy.io import wavfile
    _, data = wavfile.read(path)
    if data.dtype.kind == "i":
        data = data.astype(np.float32) / float(np.iinfo(data.dtype).max)
    elif data.dtype.kind == "u":
        data = (data.astype(np.float32) - 128.0) / 128.0
    data = data.astype(np.float32)
    return data.mean(axis=1) if data.ndim > 1 else data


def get_audio_length(path: str) -> float:
    with wave.open(path, "rb") as w:
        return w.getnframes() / float(w.getframerate())


def _wav_rate(path: str) -> int:
    with wave.open(path, "rb") as w:
        return int(w.getframerate())


def load_audio_segment(path: str, sample_rate: int, start_time: float, end_time: float) -> np.ndarray:
    """The samples between ``start_time`` and ``end_time`` (seconds) of a recording, mono, resampled to
    ``sample_rate``.  In-process counterpart of the reference's ``audio_with_sox``
    (audio_data/data_loader.py:277-289: ``sox ... trim start =end`` into a temporary file)."""
    from scipy.signal import resample
    y = load_audio(path)
    rate = _wav_rate(path)
    lo = max(int(round(start_time * rate)), 0)
    hi = min(int(round(end_time * rate)), len(y))
    seg = y[lo:max(hi, lo)]
    if rate != sample_rate and len(seg):
        seg = resample(seg, max(int(round(len(seg) * sample_rate / float(rate))), 1)).astype(np.float32)
    return seg.astype(np.float32)


audio_with_sox = load_audio_segment  # the reference's name for it


def augment_audio(path: str, sample_rate: int, tempo: float, gain: float) -> np.ndarray:
    """Tempo (speed factor) and gain (dB) applied to one recording, resampled to ``sample_rate``
    (reference: ``augment_audio_with_sox``, audio_data/data_loader.py:292-305)."""
    from scipy.signal import resample
    y = load_audio(path)
    rate = _wav_rate(path)
    n = max(int(round(len(y) / tempo * sample_rate / float(rate))), 1)
    y = resample(y, n).astype(np.float32)
    return np.clip(y * (10.0 ** (gain / 20.0)), -1.0, 1.0)


augment_audio_with_sox = augment_audio


def load_randomly_augmented_audio(path, sample_rate=16000, tempo_range=(0.85, 1.15), gain_range=(-6, 8)):
    """Random speed and gain perturbation of one utterance."""
    tempo = np.random.uniform(*tempo_range)
    gain_db = np.random.uniform(*gain_range)
    return augment_audio(path, sample_rate, tempo, gain_db)


class NoiseInjection:
    """Adds a random crop of a random noise file at a random level."""

    def __init__(self, path=None, sample_rate=16000, noise_levels=(0, 0.5)):
        if path is None or not os.path.isdir(path):
            raise IOError("Directory doesn't exist: {}".format(path))
        self.paths = sorted(os.path.join(dp, f) for dp, _, fs in os.walk(path) for f in fs if f.endswith(".wav"))
        self.sample_rate, self.noise_levels = sample_rate, noise_levels

    def inject_noise(self, data):
        return self.inject_noise_sample(data, np.random.choice(self.paths), np.random.uniform(*self.noise_levels))

    def inject_noise_sample(self, data, noise_path, noise_level):
        noise = load_audio(noise_path)
        if len(noise) < len(data):
            noise = np.tile(noise, int(math.ceil(len(data) / max(len(noise), 1))))
        start = np.random.randint(0, len(noise) - len(data) + 1)
        crop = noise[start:start + len(data)]
        ne = math.sqrt(float(crop.dot(crop)) / crop.size) + 1e-12
        de = math.sqrt(float(data.dot(data)) / data.size)
        return data + noise_level * crop * de / ne


class AudioParser:
    def parse_transcript(self, transcript_path):
        raise NotImplementedError

    def parse_audio(self, audio_path):
        raise NotImplementedError


class SpectrogramParser(AudioParser):
    def __init__(self, audio_conf, normalize=False, augment=False):
        self.window_stride, self.window_size = audio_conf["window_stride"], audio_conf["window_size"]
        self.sample_rate = audio_conf["sample_rate"]
        self.window_fn = _WINDOWS.get(audio_conf.get("window", "hamming"), torch.hamming_window)
        self.normalize, self.augment = normalize, augment
        nd = audio_conf.get("noise_dir")
        self.noiseInjector = NoiseInjection(nd, self.sample_rate, audio_conf["noise_levels"]) if nd else None
        self.noise_prob = audio_conf.get("noise_prob")

    def spectrogram(self, y: np.ndarray) -> torch.Tensor:
        n_fft = int(self.sample_rate * self.window_size)
        hop = int(self.sample_rate * self.window_stride)
        d = torch.stft(torch.from_numpy(np.ascontiguousarray(y, dtype=np.float32)), n_fft=n_fft, hop_length=hop,
                       win_length=n_fft, window=self.window_fn(n_fft, periodic=False), center=True,
                       pad_mode="reflect", return_complex=True)
        spect = torch.log1p(d.abs())
        if self.normalize:
            spect = (spect - spect.mean()) / spect.std()
        return spect

    def parse_audio(self, audio_path):
        y = load_randomly_augmented_audio(audio_path, self.sample_rate) if self.augment else load_audio(audio_path)
        if self.noiseInjector is not None and np.random.binomial(1, self.noise_prob):
            y = self.noiseInjector.inject_noise(y)
        return self.spectrogram(y)


class SpectrogramDataset(Dataset, SpectrogramParser):
    def __init__(self, audio_conf, manifest_filepath, labels, normalize=False, augment=False):
        with open(manifest_filepath) as fh:
            self.ids = [line.strip().split(",") for line in fh if line.strip()]
        self.size = len(self.ids)
        self.labels_map = {labels[i]: i for i in range(len(labels))}
        SpectrogramParser.__init__(self, audio_conf, normalize, augment)

    def __getitem__(self, index):
        audio_path, transcript_path = self.ids[index][0], self.ids[index][1]
        return self.parse_audio(audio_path), self.parse_transcript(transcript_path)

    def parse_transcript(self, transcript_path):
        with open(transcript_path, "r") as fh:
            text = fh.read().replace("\n", "")
        return [i for i in (self.labels_map.get(ch) for ch in text) if i]

    def __len__(self):
        return self.size


def collate_spectrograms(batch):
    """Pad to the longest utterance, longest first."""
    batch = sorted(batch, key=lambda s: s[0].size(1), reverse=True)
    freq, longest = batch[0][0].size(0), batch[0][0].size(1)
    inputs = torch.zeros(len(batch), 1, freq, longest)
    pct = torch.empty(len(batch), dtype=torch.float32)
    sizes = torch.empty(len(batch), dtype=torch.int32)
    targets: List[int] = []
    for i, (spect, target) in enumerate(batch):
        n = spect.size(1)
        inputs[i, 0, :, :n] = spect
        pct[i] = n / float(longest)
        sizes[i] = len(target)
        targets.extend(target)
    return inputs, torch.tensor(targets, dtype=torch.int32), pct, sizes


_collate_fn = collate_spectrograms


class AudioDataLoader(DataLoader):
    def __init__(self, *args, **kwargs):
        kwargs.setdefault("collate_fn", collate_spectrograms)
        super().__init__(*args, **kwargs)


class BucketingSampler(Sampler):
    """Batches of neighbouring (similar-length) utterances."""

    def __init__(self, data_source, batch_size=1):
        self.data_source = data_source
        ids = list(range(len(data_source)))
        self.bins = [ids[i:i + batch_size] for i in range(0, len(ids), batch_size)]

    def __iter__(self):
        for ids in self.bins:
            np.random.shuffle(ids)
            yield ids

    def __len__(self):
        return len(self.bins)

    def shuffle(self, epoch):
        np.random.shuffle(self.bins)


class DistributedBucketingSampler(Sampler):
    """Every rank takes each ``num_replicas``-th bucket, padded to equal counts."""

    def __init__(self, data_source, batch_size=1, num_replicas=None, rank=None):
        if num_replicas is None or rank is None:
            import torch.distributed as dist
            num_replicas = dist.get_world_size() if num_replicas is None else num_replicas
            rank = dist.get_rank() if rank is None else rank
        self.data_source = data_source
        self.ids = list(range(len(data_source)))
        self.batch_size = batch_size
        self.bins = [self.ids[i:i + batch_size] for i in range(0, len(self.ids), batch_size)]
        self.num_replicas, self.rank = num_replicas, rank
        self.num_samples = int(math.ceil(len(self.bins) / float(num_replicas)))
        self.total_size = self.num_samples * num_replicas
        self.epoch = 0

    def __iter__(self):
        bins = self.bins + self.bins[:self.total_size - len(self.bins)]
        return iter(bins[self.rank::self.num_replicas])

    def __len__(self):
        return self.num_samples

    def shuffle(self, epoch):
        g = torch.Generator().manual_seed(epoch)
        self.bins = [self.bins[i] for i in torch.randperm(len(self.bins), generator=g).tolist()]

    def set_epoch(self, epoch):
        self.epoch = epoch


def order_and_prune_files(file_paths, min_duration: Optional[float] = None, max_duration: Optional[float] = None):
    timed = [(p, get_audio_length(p)) for p in file_paths]
    if min_duration and max_duration:
        timed = [(p, t) for p, t in timed if min_duration <= t <= max_duration]
    return [p for p, _ in sorted(timed, key=lambda pt: pt[1])]


def create_manifest(data_path, output_path, min_duration=None, max_duration=None):
    """Write ``wav,txt`` lines for every wav under ``data_path`` (transcripts
    are expected under a sibling ``txt/`` folder), shortest first."""
    wavs = [os.path.join(dp, f) for dp, _, fs in os.walk(data_path) for f in fs if f.endswith(".wav")]
    with open(output_path, "w") as fh:
        for wav_path in order_and_prune_files(wavs, min_duration, max_duration):
            txt = wav_path.replace("/wav/", "/txt/").replace(".wav", ".txt")
            fh.write(os.path.abspath(wav_path) + "," + os.path.abspath(txt) + "\n")
