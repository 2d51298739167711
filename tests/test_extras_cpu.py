"""CPU tests of the parts around the training path: extra model families, data
preparation tools, the dependency-free dense wrapper, small utilities and the
optional-dependency gates."""
import os
import wave

import numpy as np
import pytest
import torch

from gtopkssgd_b200.utils.launch import spawn_ranks

import _workers


@pytest.mark.parametrize("factory,kw", [("preresnet20", {}), ("resnet_mod20", {}), ("resnext29_8_64", {}),
                                        ("densenet100_12", {}), ("caffe_cifar", {})])
def test_extra_cifar_models_forward(factory, kw):
    from gtopkssgd_b200.models import cifar_extras as ce
    if not hasattr(ce, factory):
        pytest.skip("no factory %s" % factory)
    net = getattr(ce, factory)(num_classes=10, **kw)
    net.eval()
    with torch.no_grad():
        out = net(torch.randn(2, 3, 32, 32))
    out = out[0] if isinstance(out, (tuple, list)) else out
    assert out.shape == (2, 10) and torch.isfinite(out).all()


@pytest.mark.parametrize("name,params", [("resnet18", 11689512), ("resnet34", 21797672), ("resnet50", 25557032)])
def test_imagenet_resnet_parameter_counts(name, params):
    from gtopkssgd_b200.models import imagenet_resnet as ir
    net = getattr(ir, name)(num_classes=1000)
    assert sum(p.numel() for p in net.parameters()) == params


def test_raw_to_wav_and_an4_manifest(tmp_path):
    from gtopkssgd_b200.data import prepare_audio as pa
    assert pa.clean_an4_transcript("<s> hello world </s> (an4-x-1)") == "HELLO WORLD"
    root = tmp_path / "an4"
    for tag, folder in (("train", "an4_clstk"), ("test", "an4test_clstk")):
        d = root / "wav" / folder / "spk"
        d.mkdir(parents=True)
        ids = []
        for i, secs in enumerate((2.0, 0.3)):  # the second clip is shorter than the 1 s floor
            samples = (np.sin(np.arange(int(16000 * secs)) * 0.05) * 8000).astype(">i2")
            samples.tofile(d / ("u%d.raw" % i))
            ids.append("%s/spk/u%d" % (folder, i))
        (root / "etc").mkdir(exist_ok=True)
        (root / "etc" / ("an4_%s.fileids" % tag)).write_text("\n".join(ids) + "\n")
        (root / "etc" / ("an4_%s.transcription" % tag)).write_text(
            "<s> one two </s> (u0)\n<s> three </s> (u1)\n")
    target = tmp_path / "out"
    pa.main(["an4", "--root", str(root), "--target", str(target)])
    with wave.open(str(target / "train" / "an4" / "wav" / "u0.wav")) as w:
        assert w.getframerate() == 16000 and w.getnframes() == 32000 and w.getsampwidth() == 2
    assert (target / "train" / "an4" / "txt" / "u0.txt").read_text() == "ONE TWO"
    train = (target / "an4_train_manifest.csv").read_text().strip().splitlines()
    val = (target / "an4_val_manifest.csv").read_text().strip().splitlines()
    assert len(train) == 1 and train[0].split(",")[0].endswith("u0.wav")   # pruned to [1, 15] seconds
    assert len(val) == 2                                                   # the test split is not pruned


def test_hdf5_converter_image_pipeline_and_gate(tmp_path):
    from PIL import Image
    from gtopkssgd_b200.data import create_hdf5 as ch
    for split in ("train", "val"):
        for cls in ("n01", "n02"):
            d = tmp_path / split / cls
            d.mkdir(parents=True)
            Image.fromarray((np.random.rand(300, 500, 3) * 255).astype(np.uint8)).save(d / "a.jpeg")
    items = ch.list_images(str(tmp_path / "train"), {"n01": 0, "n02": 1})
    assert [y for _, y in items] == [0, 1]
    img = ch.load_image(items[0][0])
    assert img.shape == (224, 224, 3) and img.dtype == np.uint8
    try:
        import h5py  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError):
            ch.convert(str(tmp_path), str(tmp_path / "x.hdf5"))
        from gtopkssgd_b200.data.datasets import DatasetHDF5
        with pytest.raises(ImportError, match="h5py"):
            DatasetHDF5(str(tmp_path / "x.hdf5"), "train")


def test_small_utilities(tmp_path, monkeypatch):
    from gtopkssgd_b200.utils import misc
    monkeypatch.chdir(tmp_path)
    assert len(misc.gen_random_id()) > 0 and misc.gen_random_id() != misc.gen_random_id()
    p = misc.create_path("a/b/c")
    assert os.path.isdir(p)
    idx, val = misc.topk(np.array([0.1, -5.0, 3.0, -0.2]), 2)
    assert set(idx.tolist()) == {1, 2} and set(val.tolist()) == {-5.0, 3.0}
    d = {}
    misc.force_insert_item(d, "k", 1)
    misc.force_insert_item(d, "k", 2)
    assert d == {"k": [1, 2]}


def test_plots_gate_and_delta_helper(tmp_path):
    from gtopkssgd_b200.analysis import plots
    for e in range(2):
        np.save(tmp_path / ("gtopknorm-rank0-epoch%d.npy" % e), np.array([1.0, 1.0]))
        np.save(tmp_path / ("randknorm-rank0-epoch%d.npy" % e), np.array([2.0, 2.0]))
    assert np.allclose(plots.delta_from_norm_files(str(tmp_path), 2), [0.25, 0.25])
    try:
        import matplotlib  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError, match="matplotlib"):
            plots.plot_delta(str(tmp_path), 2, str(tmp_path / "d.png"))
    else:
        assert os.path.isfile(plots.plot_delta(str(tmp_path), 2, str(tmp_path / "d.png")))


def test_flat_allreduce_wrapper_two_ranks():
    """The dependency-free dense wrapper: gradients are averaged over ranks,
    weights start identical."""
    out = spawn_ranks(_workers.flat_allreduce_worker, 2, timeout_s=120)
    assert torch.allclose(out[0]["grad"], out[1]["grad"]) and torch.equal(out[0]["w0"], out[1]["w0"])
    assert torch.allclose(out[0]["grad"], out[0]["expected"], atol=1e-6)


def test_deepspeech_package_roundtrip_and_description(tmp_path):
    from gtopkssgd_b200.models import lstm_models as lm
    labels = "_'ABC "
    net = lm.DeepSpeech(rnn_hidden_size=16, nb_layers=2, labels=labels, audio_conf={"sample_rate": 16000,
                        "window_size": 0.02, "window_stride": 0.01, "window": "hamming"}, bidirectional=True)
    pkg = lm.DeepSpeech.serialize(net, epoch=1, iteration=7, avg_loss=1.5, loss_results=[3.0, 2.0],
                                  cer_results=[50.0, 40.0], wer_results=[90.0, 80.0])
    path = tmp_path / "ds.pth"
    torch.save(pkg, path)
    again = lm.DeepSpeech.load_model(str(path))
    for (k, a), (_, b) in zip(net.state_dict().items(), again.state_dict().items()):
        assert torch.equal(a, b), k
    info = lm.describe_saved_model(str(path))
    assert info["rnn_layers"] == 2 and info["rnn_size"] == 16 and info["classes"] == len(labels)
    assert info["parameters"] == lm.DeepSpeech.get_param_size(net) and info["epoch"] == 2
    assert info["training"][1] == {"epoch": 2, "loss": 2.0, "wer": 80.0, "cer": 40.0}
    lm.main(["--model-path", str(path)])


def test_model_average_of_trainers(tmp_path, monkeypatch):
    from types import SimpleNamespace
    from gtopkssgd_b200.trainer.evaluate import model_average
    nets = []
    for seed in (0, 1, 2):
        torch.manual_seed(seed)
        nets.append(torch.nn.Sequential(torch.nn.Linear(5, 3), torch.nn.BatchNorm1d(3)))
    want = {k: sum(n.state_dict()[k].float() for n in nets) / 3 for k in nets[0].state_dict()}
    model_average([SimpleNamespace(net=n) for n in nets])
    for k, v in nets[0].state_dict().items():
        assert torch.allclose(v.float(), want[k].to(v.dtype).float(), atol=1e-6), k


def test_clock_sampler_parses_and_falls_back(monkeypatch):
    """Throttle reasons and the median clock come from nvidia-smi's CSV lines;
    a region too short for a periodic sample gets one query afterwards."""
    import subprocess
    from types import SimpleNamespace
    from gtopkssgd_b200.utils import timing
    line = "0, 1950, 1965, 640.5, 0x0000000000000004, Not Active, Not Active, Not Active, Active"

    class FakePopen:
        def __init__(self, *a, **k):
            self.stdout = iter([])  # the periodic sampler produced nothing

        def terminate(self):
            pass

        def wait(self, timeout=None):
            return 0

    monkeypatch.setattr(subprocess, "Popen", FakePopen)
    monkeypatch.setattr(subprocess, "run", lambda *a, **k: SimpleNamespace(stdout=line + "\n"))
    c = timing.ClockSampler(gpu_index=0, period_ms=100)
    c.start()
    out = c.stop()
    assert out["sm_mhz"] == 1950.0 and out["sm_max_mhz"] == 1965.0 and out["samples"] == 1
    assert out["reasons"] == ["sw_power_cap"] and out["power_w_max"] == 640.5


# ---- offline analysis: communication logs, fits, timelines ------------------------------------------------
def test_comm_log_readers_and_alpha_beta_fit(tmp_path):
    """Synthetic logs in the formats the paper scripts read (scripts/icdcs2019/communication.py:235-309,
    557-586, utils.py:4-53, plot_sth.py:117-136)."""
    import numpy as np
    from gtopkssgd_b200.analysis import comm_logs as cl
    from gtopkssgd_b200.analysis import cost_models as cm
    # nccl-tests table: 12 columns, size first, out-of-place time fifth
    nccl = tmp_path / "nccl.log"
    rows = ["# nThread 1 nGpus 8", "#       size         count      type   redop     time   algbw   busbw  error     time   algbw   busbw  error",
            "           8             2     float     sum    10.00    0.00    0.00  0e+00    10.0    0.00    0.00  0e+00"]
    for size in (1024, 16384, 65536, 1 << 20, 1 << 23):
        rows.append("%12d %12d     float     sum   %7.2f    1.00    1.75  0e+00   %7.2f    1.00    1.75  0e+00"
                    % (size, size // 4, 20 + size / 1e5, 21 + size / 1e5))
    nccl.write_text("\n".join(rows) + "\n")
    sizes, times = cl.read_nccl_tests_log(str(nccl))
    assert sizes == [16384, 65536, 1 << 20]           # 8 bytes, below and above the window dropped
    assert times[0] == pytest.approx(20 + 16384 / 1e5, abs=0.01)
    # MPI probe: "<size> <...> <time>", several samples per size, comments skipped
    alpha, beta = 0.436, 3.6e-5
    probe = tmp_path / "p2platency.log"
    rng = np.random.RandomState(0)
    lines = ["# size iters time", "[rank 0] warm-up"]
    for size in (16384, 65536, 262144, 1 << 20, 1 << 22):
        for _ in range(5):
            lines.append("%d 10 %.6f" % (size, (alpha + beta * size) * 1000.0 + rng.normal(0, 1e-3)))
    probe.write_text("\n".join(lines) + "\n")
    s, mean, std = cl.read_allreduce_log(str(probe))
    assert s == [16384, 65536, 262144, 1 << 20, 1 << 22] and all(x < 0.01 for x in std)
    a, b = cl.fit_alpha_beta(s, [m / 1000.0 for m in mean])
    assert a == pytest.approx(alpha, rel=1e-2) and b == pytest.approx(beta, rel=1e-3)
    pred = cl.predict_allreduce(s, 8)
    assert pred == [cm.ring_allreduce_us(8, float(m)) for m in s] and pred[0] < pred[-1]
    assert cl.relative_error(pred, pred) == 0.0
    # "<nodes>,<size> ... <time>"
    nodes = tmp_path / "nodes.log"
    nodes.write_text("# header line here\n4,1024 x 0.5000\n4,2048 x 0.7500\n")
    assert cl.read_node_allreduce_log(str(nodes)) == (4, [1024, 2048], [0.5, 0.75])
    # per-layer records and the compute-only CSV
    layers = tmp_path / "layers.log"
    layers.write_text("I0 comm [0, 1000.0, 120.0, 80.0, 90.0]\n"
                      "I0 comm [1, 2000.0, 0.4, 80.0, 90.0]\n"       # compute truncates to 0: skipped
                      "I0 comm [2, 4000000.0, 300.0, 500.0, 510.0]\n")
    sz, comms, comps, merged = cl.read_layer_log(str(layers))
    assert sz == [1000.0, 4000000.0] and comps == [120.0, 300.0] and comms == merged == [90.0, 510.0]
    st = cl.gradient_size_statistics(sz)
    assert st["layers"] == 2 and st["total"] == 4001000.0 and st["below_1m_fraction"] == 0.5
    csv = tmp_path / "p100.log"
    csv.write_text("conv1,w,100,5.0\nconv1,b,10,5.0\nfc,w,4000,9.0\n")
    raw, layer_comp, layer_size = cl.read_compute_log(str(csv))
    assert raw == [100.0, 10.0, 4000.0] and layer_comp == [5.0, 9.0] and layer_size == [110.0, 4000.0]
    # the layer log drives the timeline simulator
    sim = cm.Simulator("t", comps, sz, 4)
    assert sim.mg_wfbp().total_ms <= sim.wfbp().total_ms + 1e-9


def test_figures_render_or_say_that_matplotlib_is_missing(tmp_path):
    from gtopkssgd_b200.analysis import cost_models as cm
    from gtopkssgd_b200.analysis import plots
    sim = cm.Simulator("t", [100.0, 200.0, 50.0], [1e5, 4e6, 2e4], 4)
    tls = {"wfbp": sim.wfbp(), "single": sim.single_allreduce(), "merged": sim.mg_wfbp()}
    try:
        import matplotlib  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError, match="matplotlib"):
            plots.plot_timeline(tls, str(tmp_path / "t.png"))
        return
    out = plots.plot_timeline(tls, str(tmp_path / "t.png"))
    assert os.path.getsize(out) > 0


def test_audio_segment_and_augment(tmp_path):
    """Cropping a recording by time with resampling (the reference's audio_with_sox,
    audio_data/data_loader.py:277-289) and the tempo/gain perturbation, in process."""
    from gtopkssgd_b200.data import audio
    rate = 8000
    t = np.arange(rate * 2) / rate
    pcm = (np.sin(2 * np.pi * 440 * t) * 0.5 * 32767).astype(np.int16)
    path = str(tmp_path / "tone.wav")
    with wave.open(path, "wb") as w:
        w.setnchannels(1)
        w.setsampwidth(2)
        w.setframerate(rate)
        w.writeframes(pcm.tobytes())
    seg = audio.load_audio_segment(path, 16000, 0.5, 1.0)
    assert seg.dtype == np.float32 and abs(len(seg) - 8000) <= 1            # 0.5 s at 16 kHz
    assert 0.3 < float(np.abs(seg).max()) < 0.6
    same = audio.audio_with_sox(path, rate, 0.25, 0.75)
    assert len(same) == 4000 and np.allclose(same, audio.load_audio(path)[2000:6000])
    assert len(audio.load_audio_segment(path, rate, 1.9, 5.0)) == 800       # clipped to the end of the file
    fast = audio.augment_audio(path, rate, tempo=2.0, gain=-6.0)
    assert abs(len(fast) - rate) <= 1 and float(np.abs(fast).max()) == pytest.approx(0.25, rel=0.1)
    assert audio.augment_audio_with_sox is audio.augment_audio


def test_bench_report_tables_from_json_lines(tmp_path):
    """The tables of measured results are built from bench.py's JSON lines (both arms) and the
    micro-benchmark files; here from synthetic ones."""
    import json
    from gtopkssgd_b200.analysis import bench_report as br

    def line(value, ms, e2e, impl, comm):
        return json.dumps({"impl": impl, "value": value, "ms_per_step": ms, "e2e": {"value": e2e},
                           "comm_ms_per_iter": comm})
    for n in (1, 2):
        d = tmp_path / ("n%d" % n)
        d.mkdir()
        (d / "ours_resnet50.json").write_text("noise before\n" + line(1000.0 * n * 0.99 ** (n - 1), 64.0, 990.0 * n, "ours",
                                                                     {"select_ms": 0.05, "exchange_ms": 0.1, "exchange_wait_ms": 0.08}) + "\n")
        (d / "ref_resnet50.json").write_text(line(500.0 * n * 0.9 ** (n - 1), 128.0, 495.0 * n, "reference",
                                                  {"select_ms": 1.0, "exchange_ms": 5.0}) + "\n")
        (d / "ref_vgg16.json").write_text(json.dumps({"impl": "reference", "unavailable": "why"}) + "\n")
    (tmp_path / "n2" / "allreduce.json").write_text(json.dumps({"rows": [
        {"d": 1000000, "rho": 0.001, "k": 1000, "P": 2, "ours_ms": 0.06, "k1_ms": 0.03, "k2_ms": 0.04, "k2_chain_ms": 0.025,
         "dense_nccl_ms": 0.07, "dense_nccl_chain_ms": 0.04, "nvlink_roofline_ms": 2e-5}]}))
    (tmp_path / "n2" / "ref_allreduce.json").write_text(json.dumps({"rows": [
        {"d": 1000000, "rho": 0.001, "k": 1000, "P": 2, "select_ms": 0.3, "exchange_ms": 1.2, "total_ms": 1.5}]}))
    runs = br.Runs({1: [str(tmp_path / "n1")], 2: [str(tmp_path / "missing"), str(tmp_path / "n2")]})
    assert runs.get(1, "ref_vgg16") is None                      # an "unavailable" line is not a measurement
    text = br.report(runs)
    assert "| resnet50 | 2 | 1980 | 64.00 | 1980 | 900 | 128.00 | 990 | **2.00×** |" in text
    eff = br.efficiencies(runs)
    assert eff["ours_resnet50"][2] == pytest.approx(0.99) and eff["ref_resnet50"][2] == pytest.approx(0.9)
    assert "**P = 2**" in text and "| 1.0 M | 0.001 | 1000 | 0.030 | 0.040 / 0.025 | 0.060 / 0.055 | 0.070 / 0.040 | 0.30 + 1.20 |" in text
    assert "25×" in text                                          # reference total 1.5 ms / ours 0.06 ms
    br.main(["--runs", "1=%s" % (tmp_path / "n1"), "2=%s" % (tmp_path / "n2")])


def test_speedup_studies_and_norm_log(tmp_path):
    """scripts/icdcs2019/communication.py:350-418, 420-470, 545-555 and plot_loss.py:128-141 as numbers."""
    from gtopkssgd_b200.analysis import cost_models as cm
    from gtopkssgd_b200.analysis.log_parser import read_norm_from_log, value_histogram
    assert cm.ssgd_speedup(0.0, 8) == 8 and cm.ssgd_speedup(1.0, 8) == 4
    computes = [3000.0, 3500.0, 5000.0, 6000.0, 2000.0]
    sizes = [2e6, 5e5, 4e6, 1e5, 3e6]
    s = cm.simulated_speedups(computes, sizes, batch=32, nnodes=(4, 16))
    assert s["nodes"] == [4, 16] and all(0 < v <= n + 1e-9 for key in ("wfbp", "merged", "single") for v, n in zip(s[key], s["nodes"]))
    assert all(m >= w - 1e-9 for m, w in zip(s["merged"], s["wfbp"]))       # merging never loses to plain WFBP
    comp, comms = cm.real_comm_costs([100.0, 180.0, 320.0], batch=32)
    assert comp == pytest.approx(32 / 100.0) and comms[0] == pytest.approx(32 / 90.0 - 0.32)
    log = tmp_path / "norm.log"
    log.write_text("x INFO [rank:0][1] gtopk-dense norm mean: 0.125, std: 0.01\nother line\n"
                   "x INFO [rank:0][2] gtopk-dense norm mean: 0.1, std: 0.02\n")
    assert read_norm_from_log(str(log)) == ([0.125, 0.1], [0.01, 0.02])
    h = value_histogram([-1.0, 0.0, 1.0, 3.0], bins=4)
    assert h["non_positive"] == 2 and h["total"] == 4 and h["mean"] == 0.75 and len(h["density"]) == 4
