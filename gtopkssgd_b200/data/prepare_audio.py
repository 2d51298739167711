"""Build AN4 / LibriSpeech manifests from locally extracted corpora
(reference: audio_data/an4.py, audio_data/librispeech.py, audio_data/utils.py;
those scripts also download the archives and shell out to sox -- here the
archives must already be on disk and conversion is done in-process).

    python -m gtopkssgd_b200.data.prepare_audio an4 --root an4/ --target an4_dataset/
    python -m gtopkssgd_b200.data.prepare_audio librispeech --root LibriSpeech/train-clean-100 --target libri/ --name train

Output: ``<target>/<name>/wav/*.wav``, ``<target>/<name>/txt/*.txt`` and a
manifest CSV ``wav path,txt path`` sorted by duration (optionally pruned to
[min, max] seconds).  LibriSpeech FLAC input needs the ``soundfile`` package.
"""
from __future__ import annotations

import argparse
import os
import wave

import numpy as np

from .audio import create_manifest


def raw_to_wav(raw_path, wav_path, sample_rate=16000, big_endian=True):
    data = np.fromfile(raw_path, dtype=">i2" if big_endian else "<i2").astype("<i2")
    with wave.open(wav_path, "wb") as w:
        w.setnchannels(1)
        w.setsampwidth(2)
        w.setframerate(sample_rate)
        w.writeframes(data.tobytes())


def clean_an4_transcript(line: str) -> str:
    return line.split("(")[0].strip("<s>").split("<")[0].strip().upper()


def prepare_an4(root, target, min_duration=1, max_duration=15):
    for tag, folder, prune in (("train", "an4_clstk", True), ("test", "an4test_clstk", False)):
        wav_dir, txt_dir = os.path.join(target, tag, "an4", "wav"), os.path.join(target, tag, "an4", "txt")
        os.makedirs(wav_dir, exist_ok=True)
        os.makedirs(txt_dir, exist_ok=True)
        with open(os.path.join(root, "etc", "an4_%s.fileids" % tag)) as fh:
            ids = [l.strip() for l in fh if l.strip()]
        with open(os.path.join(root, "etc", "an4_%s.transcription" % tag)) as fh:
            texts = [clean_an4_transcript(l) for l in fh]
        for fid, text in zip(ids, texts):
            name = os.path.basename(fid)
            raw_to_wav(os.path.join(root, "wav", fid + ".raw"), os.path.join(wav_dir, name + ".wav"))
            with open(os.path.join(txt_dir, name + ".txt"), "w") as out:
                out.write(text)
        manifest = os.path.join(target, "an4_%s_manifest.csv" % ("train" if tag == "train" else "val"))
        create_manifest(os.path.join(target, tag), manifest, min_duration if prune else None,
                        max_duration if prune else None)
        print("wrote", manifest)


def prepare_librispeech(root, target, name, min_duration=1, max_duration=15, sample_rate=16000):
    import soundfile as sf
    wav_dir, txt_dir = os.path.join(target, name, "wav"), os.path.join(target, name, "txt")
    os.makedirs(wav_dir, exist_ok=True)
    os.makedirs(txt_dir, exist_ok=True)
    for dp, _, files in os.walk(root):
        for trans in (f for f in files if f.endswith(".trans.txt")):
            with open(os.path.join(dp, trans)) as fh:
                for line in fh:
                    uid, text = line.strip().split(" ", 1)
                    audio, sr = sf.read(os.path.join(dp, uid + ".flac"), dtype="int16")
                    if sr != sample_rate:
                        raise ValueError("unexpected sample rate %d in %s" % (sr, uid))
                    with wave.open(os.path.join(wav_dir, uid + ".wav"), "wb") as w:
                        w.setnchannels(1)
                        w.setsampwidth(2)
                        w.setframerate(sr)
                        w.writeframes(np.asarray(audio, dtype="<i2").tobytes())
                    with open(os.path.join(txt_dir, uid + ".txt"), "w") as out:
                        out.write(text.upper())
    manifest = os.path.join(target, "libri_%s_manifest.csv" % name)
    create_manifest(os.path.join(target, name), manifest, min_duration, max_duration)
    print("wrote", manifest)


def main(argv=None):
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="corpus", required=True)
    a = sub.add_parser("an4")
    a.add_argument("--root", required=True)
    a.add_argument("--target", default="an4_dataset/")
    a.add_argument("--min-duration", type=int, default=1)
    a.add_argument("--max-duration", type=int, default=15)
    b = sub.add_parser("librispeech")
    b.add_argument("--root", required=True)
    b.add_argument("--target", default="LibriSpeech_dataset/")
    b.add_argument("--name", default="train")
    b.add_argument("--min-duration", type=int, default=1)
    b.add_argument("--max-duration", type=int, default=15)
    args = ap.parse_args(argv)
    if args.corpus == "an4":
        prepare_an4(args.root, args.target, args.min_duration, args.max_duration)
    else:
        prepare_librispeech(args.root, args.target, args.name, args.min_duration, args.max_duration)


if __name__ == "__main__":
    main()
