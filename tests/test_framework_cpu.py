"""CPU tests of the framework layers: grouping, density schedule, compressor
API, LR schedules, checkpoints + evaluate, log formats, models, data."""
import math
import os
import re
import time

import numpy as np
import pytest
import torch

from gtopkssgd_b200 import settings
from gtopkssgd_b200.models import create_net
from gtopkssgd_b200.parallel.compression import TopKCompressor, compressors
from gtopkssgd_b200.parallel.distributed_optimizer import DistributedOptimizer
from gtopkssgd_b200.parallel.flat_buffer import FlatBuffers, generate_groups


def test_model_sizes_match_the_reference_table():
    expected = {"resnet20": (269722, 59), "resnet56": (853018, 167), "resnet110": (1727962, 329),
                "vgg16": (14728266, 54), "resnet50": (25557032, 161), "alexnet": (61100840, 16)}
    for dnn, (numel, ntensors) in expected.items():
        net, _ = create_net(1000 if dnn in ("resnet50", "alexnet") else 10, dnn)
        ps = list(net.parameters())
        assert (sum(p.numel() for p in ps), len(ps)) == (numel, ntensors), dnn
    net, _ = create_net(10, "lstm", vocab_size=10000, batch_size=20)
    assert sum(p.numel() for p in net.parameters()) == 66034000
    net, ext = create_net(29, "lstman4")
    assert sum(p.numel() for p in net.parameters()) == 27569568 and len(ext["labels"]) == 29


def test_state_dict_keys_are_reference_compatible():
    net, _ = create_net(10, "resnet20")
    keys = set(net.state_dict())
    for k in ("conv_1_3x3.weight", "bn_1.running_mean", "stage_1.0.conv_a.weight", "stage_3.2.bn_b.bias",
              "classifier.weight"):
        assert k in keys
    net, _ = create_net(10, "vgg16")
    assert {"features.0.weight", "features.1.running_var", "fc.bias"} <= set(net.state_dict())
    net, _ = create_net(1000, "resnet50")
    assert {"conv1.weight", "layer1.0.downsample.0.weight", "layer4.2.bn3.weight", "fc.weight"} <= set(net.state_dict())


def test_grouping_by_threshold_backward_order():
    names = ["a", "b", "c", "d", "e"]
    sizes = dict(zip(names, [10, 20, 30, 40, 50]))
    groups, key_group = generate_groups(names, sizes, 60)
    assert groups == [["e", "d"], ["c", "b", "a"]]  # last layer first; a group closes once it holds >= 60
    assert key_group == {"e": 0, "d": 0, "c": 1, "b": 1, "a": 1}
    groups, _ = generate_groups(names, sizes, 640 * 1024 * 1024)
    assert groups == [["e", "d", "c", "b", "a"]]  # default: the whole model is one group


def test_flat_buffers_keep_views_and_values():
    net, _ = create_net(10, "resnet20")
    before = {n: p.detach().clone() for n, p in net.named_parameters()}
    fb = FlatBuffers(net.named_parameters(), 100000)
    assert len(fb.groups) == 3 and fb.param_numel == 269722
    assert all(s.offset % 4 == 0 for s in fb.slots.values())  # every parameter view is 16-byte aligned
    for n, p in net.named_parameters():
        assert torch.equal(p, before[n])
        s = fb.slots[n]
        assert p.data_ptr() == fb.param.data_ptr() + 4 * s.offset
    net(torch.randn(2, 3, 32, 32)).sum().backward()
    assert float(fb.grad.abs().sum()) > 0
    for p in net.parameters():
        p.grad = None  # what zero_grad(set_to_none=True) does
    assert fb.ensure_views() == 59


def test_density_schedule_and_pin(monkeypatch):
    net, _ = create_net(10, "mnistnet")
    opt = torch.optim.SGD(net.parameters(), lr=0.1)
    monkeypatch.setattr(settings, "PIN_DENSITY", False)
    d = DistributedOptimizer(opt, net.named_parameters(), compression=compressors["gtopk"], is_sparse=True,
                             density=0.001)
    assert d.get_current_density() == 0.004  # epoch 0
    d.add_train_epoch()
    assert d.get_current_density() == 0.001
    d.stop()
    monkeypatch.setattr(settings, "PIN_DENSITY", True)
    d = DistributedOptimizer(opt, net.named_parameters(), compression=compressors["gtopk"], is_sparse=True,
                             density=0.001)
    assert d.get_current_density() == 0.001
    d.stop()


def test_compressor_registry_api():
    assert set(compressors) == {"topk", "topk2", "gtopk", "none"}
    TopKCompressor.clear()
    torch.manual_seed(0)
    t = torch.randn(1000)
    orig = t.clone()
    out, idx = compressors["gtopk"].compress(t, "g0", ratio=0.01)
    assert out is t and idx.numel() == 10
    assert int((t != 0).sum()) == 10 and torch.equal(t[idx], orig[idx])
    res = TopKCompressor.get_residuals("g0", t)
    assert torch.allclose(res + t, orig)
    # positions 0 and 1 of the selection were accepted globally, the rest returns to the residual
    compressors["gtopk"].add_residuals(np.array([0, 1]), "g0")
    back = idx[2:]
    assert torch.allclose(res[back], orig[back]) and float(res[idx[:2]].abs().sum()) == 0
    dense, ctx = compressors["none"].compress(t, "x", sigma_scale=2.5, ratio=0.5)
    assert dense is t and ctx is None
    TopKCompressor.clear()


def test_gradient_accumulation_local_flag(monkeypatch):
    monkeypatch.setattr(settings, "PIN_DENSITY", True)
    torch.manual_seed(0)
    net, _ = create_net(10, "mnistnet")
    net.eval()  # no dropout noise
    opt = torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.9)
    d = DistributedOptimizer(opt, net.named_parameters(), compression=compressors["gtopk"], is_sparse=True,
                             density=0.01)
    x = torch.randn(4, 1, 28, 28)
    d.zero_grad()
    d.local = True
    net(x).sum().backward()
    assert d._allreducer.allreduce_count == 0  # hooks skipped on the accumulation micro-step
    d.local = False
    net(x).sum().backward()
    assert d._allreducer.allreduce_count == 1
    d.step()
    d.stop()


def _tiny_trainer(tmp_path, monkeypatch, **kw):
    from gtopkssgd_b200.trainer.dl_trainer import DLTrainer
    monkeypatch.chdir(tmp_path)
    args = dict(dist=False, ngpus=0, batch_size=4, data_dir="synthetic", dataset="cifar10", dnn="resnet20", lr=0.1,
                nworkers=1, synthetic_train_size=64)
    args.update(kw)
    return DLTrainer(0, 1, **args)


def test_lr_schedules(tmp_path, monkeypatch):
    t = _tiny_trainer(tmp_path, monkeypatch, nworkers=4)
    t.num_batches_per_epoch = 100
    t.train_iter = 0
    assert t.adjust_learning_rate(0, t.optimizer) == pytest.approx(0.1 / 4)  # warm-up starts at base_lr / P
    t.train_iter = 500
    assert t.adjust_learning_rate(5, t.optimizer) == pytest.approx(0.025 + 0.075 * 0.5)
    for epoch, scale in ((10, 1.0), (80, 1.0), (81, 0.1), (121, 0.1), (122, 0.01), (155, 0.001)):
        assert t.adjust_learning_rate(epoch, t.optimizer) == pytest.approx(0.1 * scale)
    t.dataset = "imagenet"
    for epoch, scale in ((29, 1.0), (30, 0.1), (60, 0.01), (80, 0.001)):
        assert t.adjust_learning_rate(epoch, t.optimizer) == pytest.approx(0.1 * scale)
    t.dnn = "lstm"
    for epoch, scale in ((0, 1.0), (62, 1.0), (63, 0.01), (79, 0.01), (80, 0.001)):
        assert t.adjust_learning_rate(epoch, t.optimizer) == pytest.approx(0.1 * scale)
    t.dnn, t.lstman4_lr_epoch_tag, t.train_iter = "lstman4", 0, 100
    t._set_lr(t.optimizer, 0.0003)
    t.adjust_learning_rate(0, t.optimizer)
    assert t.lr == pytest.approx(0.0003 / 1.01)


def test_sgd_hyper_parameters_per_dataset(tmp_path, monkeypatch):
    t = _tiny_trainer(tmp_path, monkeypatch)
    g = t.optimizer.param_groups[0]
    assert (g["momentum"], g["weight_decay"], g["nesterov"]) == (0.9, 1e-4, False)
    t = _tiny_trainer(tmp_path, monkeypatch, dataset="ptb", dnn="lstm", batch_size=2, num_steps=5)
    g = t.optimizer.param_groups[0]
    assert (g["momentum"], g["weight_decay"]) == (0.0, 0.0)


def test_checkpoint_roundtrip_and_evaluate(tmp_path, monkeypatch, caplog):
    from gtopkssgd_b200.trainer import evaluate as ev
    t = _tiny_trainer(tmp_path, monkeypatch, save_checkpoints=True, prefix="unit")
    for _ in range(t.num_batches_per_epoch + 1):  # crosses one epoch boundary -> test() + checkpoint
        t.optimizer.zero_grad()
        t.train(1)
        t.update_model()
    path = os.path.join("weights", "unit", "resnet20-n1-bs4-lr0.1000", "resnet20-rank0-epoch0.pth")
    assert os.path.isfile(path)
    ckpt = torch.load(path, weights_only=False)
    assert set(ckpt) == {"iter", "epoch", "state"} and ckpt["epoch"] == 0 and ckpt["iter"] == 16
    # a dict shaped like the reference's loads into a fresh trainer
    t2 = _tiny_trainer(tmp_path, monkeypatch)
    t2.load_model_from_file(path)
    assert t2.get_train_epoch() == 0 and t2.get_train_iter() == 16
    for k, v in t2.net.state_dict().items():
        assert torch.equal(v, ckpt["state"][k])
    # evaluate.py parses dnn / batch size / lr from the directory name
    os.rename(path, os.path.join(os.path.dirname(path), "resnet20-rank0-epoch1.pth"))
    best = ev.evaluate(os.path.dirname(path), "resnet20", "cifar10", "synthetic", 1)
    assert 0.0 <= best <= 1.0
    assert ev.parse_model_dir("weights/x/resnet20-n4-bs32-lr0.1000") == ("resnet20", 32, 0.1)


def test_log_lines_match_the_reference_parsers(tmp_path, monkeypatch):
    """Regexes equivalent to the ones in scripts/*/plot_loss.py."""
    import io
    import logging
    buf = io.StringIO()
    h = logging.StreamHandler(buf)
    h.setFormatter(settings.formatter)
    settings.logger.addHandler(h)
    try:
        t = _tiny_trainer(tmp_path, monkeypatch)
        for _ in range(t.num_batches_per_epoch + 1):
            t.optimizer.zero_grad()
            t.train(1)
            t.update_model()
        settings.logger.info("Time per iteration including communication: %f. Speed: %f images/s, current density: %f",
                             0.5, 64.0, 0.001)
    finally:
        settings.logger.removeHandler(h)
    text = buf.getvalue()
    assert re.search(r"Epoch \d+, avg train acc: [\d.naN]+, lr: [\d.]+, avg loss: [\d.]+", text)
    assert re.search(r"Epoch \d+, lr: [\d.]+, val loss: [\d.]+, val acc: [\d.]+", text)
    assert re.search(r"Time per iteration including communication: [\d.]+. Speed: [\d.]+ images/s", text)
    assert re.search(r"\d{4}-\d\d-\d\d .* \[dl_trainer.py:\d+\] INFO", text)


def test_update_nworker_reshards(tmp_path, monkeypatch):
    t = _tiny_trainer(tmp_path, monkeypatch, nworkers=1)
    n1 = t.num_batches_per_epoch
    t.update_nworker(2, 1)
    assert t.nworkers == 2 and t.rank == 1 and t.num_batches_per_epoch == math.ceil(n1 / 2)
    assert t.train_sampler.num_replicas == 2 and t.train_sampler.rank == 1
    x, y = t.data_iter()
    assert x.shape == (4, 3, 32, 32)


def test_compat_functions_single_process():
    from gtopkssgd_b200.parallel import compat
    rng = np.random.RandomState(0)
    dense = rng.randn(10000).astype(np.float32)
    idx, vals = compat.topk(dense, 10)
    assert np.all(np.abs(vals)[:-1] <= np.abs(vals)[1:])  # ascending magnitude, as the reference's utils.topk
    v, i, inc = compat.gtopk_sparse_allreduce(None, vals, indexes=idx)
    assert set(i.tolist()) == set(idx.tolist()) and len(inc) == 10
    v1, i1, none = compat.topk_sparse_allreduce(None, vals, {}, indexes=idx)
    assert none is None and len(v1) == 10
    assert np.allclose(compat.dense_allreduce(None, dense), dense)
    # half-precision wire type of the all-gather variant (allreducer.py:19-24, 52-53)
    v16, i16, _ = compat.topk_sparse_allreduce(None, vals, {}, indexes=idx, dtype=np.float16)
    assert v16.dtype == np.float16 and np.array_equal(i16, i1)
    assert np.allclose(v16.astype(np.float32), vals, rtol=1e-3, atol=1e-4)


def test_ptb_reader_windows(tmp_path):
    from gtopkssgd_b200.data import ptb_reader
    words = " ".join("w%d" % (i % 17) for i in range(400))
    for part in ("train", "valid", "test"):
        (tmp_path / ("ptb.%s.txt" % part)).write_text(" " + words + " \n " + words + " \n")
    train, valid, test, w2i, i2w = ptb_reader.ptb_raw_data(str(tmp_path))
    assert len(w2i) == 18 and "<eos>" in w2i
    ds = ptb_reader.TrainDataset(train, batch_size=4, num_steps=5)
    x, y = ds[3]
    assert list(x[1:]) == list(y[:-1]) and len(ds) % 4 == 0


def test_ctc_decoders_and_error_rates():
    from gtopkssgd_b200.data.decoder import BeamCTCDecoder, GreedyDecoder, edit_distance
    labels = "_'ABCDEFGHIJKLMNOPQRSTUVWXYZ "
    dec = GreedyDecoder(labels)
    assert edit_distance("kitten", "sitting") == 3
    assert dec.wer("the cat sat", "the cat sat down") == 1 and dec.cer("abc d", "abd") == 1
    # frames: H H _ I I ' ' T -> "HI T" after collapsing repeats and blanks
    seq = [labels.index(c) for c in "HH_II T"]
    probs = torch.full((1, len(seq), len(labels)), -5.0)
    for t, c in enumerate(seq):
        probs[0, t, c] = 5.0
    strings, offsets = dec.decode(probs.softmax(-1), torch.tensor([len(seq)]))
    assert strings[0][0] == "HI T" and offsets[0][0].tolist() == [0, 3, 5, 6]
    beam = BeamCTCDecoder(labels, beam_width=8)
    out, _ = beam.decode(probs.softmax(-1), torch.tensor([len(seq)]))
    assert out[0][0] == "HI T"


def test_audio_collate_and_bucketing():
    from gtopkssgd_b200.data.audio import BucketingSampler, DistributedBucketingSampler, collate_spectrograms
    from gtopkssgd_b200.data.synthetic import SyntheticAN4
    ds = SyntheticAN4(20, 29, min_t=50, max_t=90)
    batch = [ds[i] for i in range(4)]
    inputs, targets, pct, sizes = collate_spectrograms(batch)
    assert inputs.shape[:3] == (4, 1, 161) and inputs.shape[3] == max(b[0].size(1) for b in batch)
    assert float(pct.max()) == 1.0 and int(sizes.sum()) == targets.numel()
    assert len(BucketingSampler(ds, batch_size=8)) == 3
    s0 = DistributedBucketingSampler(ds, batch_size=4, num_replicas=2, rank=0)
    s1 = DistributedBucketingSampler(ds, batch_size=4, num_replicas=2, rank=1)
    assert len(s0) == len(s1) == 3
    seen = [tuple(b) for b in s0] + [tuple(b) for b in s1]
    assert len(set(seen)) == 5  # 5 buckets, one repeated to even out the ranks


def test_lstm_and_an4_models_train_one_step():
    from gtopkssgd_b200.models.lstm import repackage_hidden
    net, _ = create_net(10, "lstm", vocab_size=50, batch_size=3, num_steps=4)
    net.embedding_dim  # noqa: B018
    h = net.init_hidden()
    x = torch.randint(0, 50, (4, 3))
    small = type(net)(50, embedding_dim=16, num_steps=4, batch_size=3)
    out, h2 = small(x, small.init_hidden())
    assert out.shape == (4, 3, 50)
    out.sum().backward()
    assert all(t.grad_fn is None for t in repackage_hidden(h2))
    del h
    from gtopkssgd_b200.models.lstm_models import DeepSpeech
    ds = DeepSpeech(labels="_ab ", rnn_hidden_size=16, nb_layers=2, bidirectional=False, context=3,
                    audio_conf={"sample_rate": 16000, "window_size": 0.02})
    y, lens = ds(torch.randn(2, 1, 161, 40), torch.tensor([40, 30]))
    assert y.shape[0] == 2 and y.shape[2] == 4 and lens.tolist() == [20, 15]
    pkg = DeepSpeech.serialize(ds, epoch=1)
    ds2 = DeepSpeech.load_model_package(pkg)
    assert pkg["epoch"] == 2 and set(ds2.state_dict()) == set(ds.state_dict())


def test_cost_models_and_simulator():
    from gtopkssgd_b200.analysis import cost_models as cm
    m, rho = 25 * 1024 * 1024, 0.001
    assert cm.gtopk_allreduce_ms(32, m, rho) < cm.topk_allreduce_ms(32, m, rho) < cm.dense_allreduce_ms(32, m)
    assert cm.gtopk_allreduce_ms(4, m, rho) > cm.topk_allreduce_ms(4, m, rho)  # the tree only pays off at scale
    eff = cm.scaling_efficiency(cm.PUBLISHED_THROUGHPUT["ResNet-50"]["gtopk"])
    assert eff[-1] == pytest.approx(100 * 39.119 / 52.873)
    assert cm.speedup_over(cm.PUBLISHED_THROUGHPUT["VGG-16"]["gtopk"],
                           cm.PUBLISHED_THROUGHPUT["VGG-16"]["dense"])[-1] == pytest.approx(9.78, abs=0.01)
    assert sum(cm.breakdown_ratios("AlexNet")) == pytest.approx(1.0)
    # three layers whose all-reduce is latency dominated: merging must not be slower than plain WFBP,
    # and both beat a single all-reduce after backward only when overlap exists
    sim = cm.Simulator("toy", computes=[100.0, 100.0, 100.0], sizes=[1000, 1000, 1000], num_of_nodes=8)
    plain, merged, single = sim.wfbp(), sim.mg_wfbp(), sim.single_allreduce()
    assert merged.total_ms <= plain.total_ms + 1e-9
    assert single.total_ms * 1000 == pytest.approx(300.0 + cm.ring_allreduce_us(8, 3000))
    assert len(plain.comm) == 3 and plain.comm[0][0] == 100.0


def test_log_parser_reads_trainer_lines(tmp_path):
    from gtopkssgd_b200.analysis.log_parser import mean_speed, parse_log
    text = "\n".join([
        "2026-01-01 10:00:00,123 [dl_trainer.py:142] INFO num_batches_per_epoch: 391",
        "2026-01-01 10:05:00,000 [dl_trainer.py:300] INFO Epoch 1, avg train acc: 35.500000, lr: 0.100000, avg loss: 1.750000",
        "2026-01-01 10:05:10,000 [dl_trainer.py:420] INFO Epoch 0, lr: 0.100000, val loss: 1.600000, val acc: 0.412000",
        "2026-01-01 10:06:00,000 [gtopk_trainer.py:120] INFO Time per iteration including communication: 0.050000. "
        "Speed: 640.000000 images/s, current density: 0.001000",
        "2026-01-01 10:07:00,000 [allreducer.py:330] INFO [rank:0]cla...ght[269722]: 0.0,0.0,0.000120,0.000250,0.0,0.0,0.0",
        "2026-01-01 10:10:00,000 [dl_trainer.py:300] INFO Epoch 2, avg train acc: 48.000000, lr: 0.100000, avg loss: 1.400000",
    ])
    p = tmp_path / "run.log"
    p.write_text(text + "\n")
    log = parse_log(str(p))
    assert log.num_batches_per_epoch == 391 and log.epochs == [1, 2]
    assert log.train_loss == [1.75, 1.4] and log.times_s == [0, 300]
    assert log.val_acc == [0.412] and log.densities == [0.001]
    assert mean_speed(log, skip=0) == 640.0
    assert log.profiling[0]["compression"] == pytest.approx(1.2e-4) and log.profiling[0]["size"] == 269722


def test_norm_clip_before_compression_and_momentum_correction(monkeypatch):
    """norm_clip scales the merged gradient to sqrt(1/P)*norm_clip before it is
    sparsified (allreducer.py:531-538 in the reference); momentum correction
    sparsifies the velocity instead of the raw gradient."""
    monkeypatch.setattr(settings, "PIN_DENSITY", True)
    torch.manual_seed(0)
    net, _ = create_net(10, "mnistnet")
    net.eval()
    opt = torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.9)
    d = DistributedOptimizer(opt, net.named_parameters(), compression=compressors["gtopk"], is_sparse=True,
                             density=1.0, norm_clip=0.5)
    x = torch.randn(4, 1, 28, 28)
    d.zero_grad()
    net(x).sum().backward()
    raw = d._flat.grad[:d._flat.numel].clone()
    assert float(raw.norm()) > 0.5
    idx, val = d._allreducer.engines[0].selector.pairs()  # density 1: everything selected, after clipping
    assert float(val.norm()) == pytest.approx(0.5, rel=1e-4)
    d.step()
    d.stop()
    # momentum correction: velocity buffer is updated in the hook and replaces the gradient
    net2, _ = create_net(10, "mnistnet")
    net2.eval()
    opt2 = torch.optim.SGD(net2.parameters(), lr=0.1, momentum=0.9)
    d2 = DistributedOptimizer(opt2, net2.named_parameters(), compression=compressors["gtopk"], is_sparse=True,
                              density=1.0)
    d2.momentum_correction = True
    p0 = d2._flat.param.clone()
    for _ in range(2):
        d2.zero_grad()
        net2(x).sum().backward()
        d2.step()
    assert float(d2._flat.momentum.abs().sum()) > 0
    assert not torch.equal(d2._flat.param, p0)
    d2.stop()


def test_profiling_norm_diagnostic(monkeypatch):
    monkeypatch.setattr(settings, "PIN_DENSITY", True)
    monkeypatch.setattr(settings, "PROFILING_NORM", True)
    net, _ = create_net(10, "mnistnet")
    net.eval()
    opt = torch.optim.SGD(net.parameters(), lr=0.01)
    d = DistributedOptimizer(opt, net.named_parameters(), compression=compressors["gtopk"], is_sparse=True,
                             density=0.01)
    d.zero_grad()
    net(torch.randn(4, 1, 28, 28)).sum().backward()
    d.step()
    (gtopk_norm, randk_norm, upbound, xnorm, std), = d._allreducer._profiling_norms
    assert 0 <= gtopk_norm <= randk_norm <= xnorm  # top-k keeps at least as much mass as random-k
    d.stop()


@pytest.mark.parametrize("dnn,dataset,extra", [("mnistnet", "mnist", []), ("lstm", "ptb", ["--num-steps", "5"])])
def test_single_gpu_cli_smoke(tmp_path, monkeypatch, dnn, dataset, extra):
    from gtopkssgd_b200.trainer import dl_trainer
    monkeypatch.chdir(tmp_path)
    dl_trainer.main(["--dnn", dnn, "--dataset", dataset, "--data-dir", "synthetic", "--batch-size", "4",
                     "--lr", "0.01", "--max-epochs", "1", "--max-iters", "2"] + extra)
    assert any(f.endswith(".log") for _, _, fs in os.walk(tmp_path / "logs") for f in fs)


def test_gtopk_cli_smoke_an4_synthetic(tmp_path, monkeypatch):
    from gtopkssgd_b200.trainer import gtopk_trainer
    monkeypatch.chdir(tmp_path)
    gtopk_trainer.main(["--dnn", "lstman4", "--dataset", "an4", "--data-dir", "synthetic", "--batch-size", "2",
                        "--lr", "0.0003", "--compression", "--compressor", "gtopk", "--density", "0.001",
                        "--max-epochs", "1", "--max-iters", "1"])
    logdir = tmp_path / "logs"
    assert any("lstman4-n1-bs2-lr0.0003-ns1-sg2.50-ds0.001" in dp for dp, _, _ in os.walk(logdir))


def test_nvtx_ranges_follow_the_switch(monkeypatch):
    """With settings.NVTX on, every timed phase and every train step is wrapped
    in a balanced NVTX range; with it off nothing is pushed."""
    from gtopkssgd_b200.utils import timing
    events = []
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda.nvtx, "range_push", lambda name: events.append(("push", name)))
    monkeypatch.setattr(torch.cuda.nvtx, "range_pop", lambda: events.append(("pop", None)))
    t = timing.PhaseTimers(enabled=False)
    t.start("g", "compression")
    t.stop("g", "compression")
    assert events == []
    monkeypatch.setattr(settings, "NVTX", True)
    t.start("g", "compression")
    with timing.nvtx_range("gtopk/train_step"):
        pass
    t.stop("g", "compression")
    assert events == [("push", "gtopk/compression"), ("push", "gtopk/train_step"), ("pop", None), ("pop", None)]


def test_stream_watchdog_reports_a_stuck_iteration_once():
    import time
    from gtopkssgd_b200.parallel.elastic import StreamWatchdog

    class FakeEvent:
        def __init__(self, done_after=None):
            self.t0, self.done_after, self.queries = time.monotonic(), done_after, 0

        def query(self):
            self.queries += 1
            return self.done_after is not None and time.monotonic() - self.t0 >= self.done_after

    stalls = []
    w = StreamWatchdog(0.2, stalls.append, poll_s=0.02)
    try:
        w.arm(FakeEvent(done_after=0.05))          # completes in time
        time.sleep(0.4)
        assert stalls == []
        stuck = FakeEvent()
        w.arm(stuck)                               # never completes
        time.sleep(0.5)
        assert len(stalls) == 1 and stalls[0] > 0.2 and w.stalls == 1
        w.pause()                                  # graph capture: no query while paused, and arming is dropped
        n = stuck.queries
        w.arm(stuck)
        w.pause()
        time.sleep(0.1)
        assert stuck.queries == n and len(stalls) == 1
        w.resume()
    finally:
        w.stop()


def test_transport_choice():
    from gtopkssgd_b200.parallel.comm import choose_transport
    one = ["a"] * 4
    assert choose_transport("auto", one, [True] * 4) == "p2p"
    assert choose_transport("auto", one, [True, True, False, True]) == "staged"      # no peer access somewhere
    assert choose_transport("auto", ["a", "a", "b", "b"], [True] * 4) == "staged"    # two hosts
    assert choose_transport("staged", one, [True] * 4) == "staged"
    with pytest.raises(RuntimeError):
        choose_transport("p2p", ["a", "b"], [True, True])
    with pytest.raises(ValueError):
        choose_transport("rdma", one, [True] * 4)


def test_resume_restores_velocity_and_residuals_through_the_wrapper(tmp_path, monkeypatch):
    """A full checkpoint written by a wrapped trainer is loaded before the new
    trainer's optimizer is wrapped; velocity and residuals must still arrive in
    the flat buffers, and the next step must equal the uninterrupted run's."""
    monkeypatch.setattr(settings, "PIN_DENSITY", True)

    def wrapped(pretrain=None):
        t = _tiny_trainer(tmp_path, monkeypatch, dnn="mnistnet", dataset="mnist", pretrain=pretrain)
        t.net.eval()  # no dropout noise: both runs see the same function
        d = DistributedOptimizer(t.optimizer, t.net.named_parameters(), compression=compressors["gtopk"],
                                 is_sparse=True, density=0.01)
        t.update_optimizer(d)
        return t, d

    g = torch.Generator().manual_seed(5)
    batches = [(torch.randn(4, 1, 28, 28, generator=g), torch.randint(0, 10, (4,), generator=g)) for _ in range(4)]
    t, d = wrapped()
    for b in batches[:3]:
        t.train_step(data=b)
    path = str(tmp_path / "full.pth")
    t.save_checkpoint(t.make_checkpoint(full=True), path)
    mom, res = d._flat.momentum.clone(), d._flat.residual.clone()
    assert float(mom.abs().sum()) > 0 and float(res.abs().sum()) > 0
    t.train_step(data=batches[3])
    want = d._flat.param.clone()
    d.stop()

    t2, d2 = wrapped(pretrain=path)
    assert t2.get_train_iter() == 3
    assert torch.equal(d2._flat.momentum, mom) and torch.equal(d2._flat.residual, res)
    t2.train_step(data=batches[3])
    assert torch.allclose(d2._flat.param, want, rtol=1e-6, atol=1e-7)
    d2.stop()


def test_group_size_limit_is_checked():
    """int32 indices: a merged group of 2^31 elements or more is refused with a hint."""
    from types import SimpleNamespace
    from gtopkssgd_b200.parallel.allreducer import GroupEngine
    from gtopkssgd_b200.parallel.flat_buffer import MergedGroup
    g = MergedGroup(0, ["w"], 0, 2 ** 31, [0], "w", 2 ** 31)
    fb = SimpleNamespace(grad=torch.zeros(1), residual=None, device=torch.device("cpu"),
                         group_slice=lambda buf, grp: buf)
    with pytest.raises(ValueError, match="2\\^31"):
        GroupEngine(SimpleNamespace(flat=fb, mode="gtopk"), g)


def test_watchdog_note_is_raised_on_the_training_thread(monkeypatch):
    """A stall seen by the watchdog thread is only noted there; err_handler and
    GTopkTimeout happen at the next pre_iteration() of the training thread."""
    from gtopkssgd_b200.parallel.allreducer import GTopkTimeout
    monkeypatch.setattr(settings, "PIN_DENSITY", True)
    net, _ = create_net(10, "mnistnet")
    calls = []
    opt = torch.optim.SGD(net.parameters(), lr=0.01)
    d = DistributedOptimizer(opt, net.named_parameters(), compression=compressors["gtopk"], is_sparse=True,
                             density=0.01, err_handler=lambda n, r: calls.append((n, r)))
    d._on_stall(123.0)
    assert calls == [] and d._stalled is not None
    with pytest.raises(GTopkTimeout, match="still running after 123 s"):
        d.zero_grad()
    assert calls == [(1, 0)]
    d.zero_grad()  # the note is consumed
    d.stop()


def test_decode_k2_trace_roles_and_wait_accounting():
    """The device-side stamps of the exchange kernel decoded into wait and work (pure host code)."""
    from gtopkssgd_b200.ops.exchange import decode_k2_trace
    # rank 0 of 4: receiver in rounds 0 and 1, then writes the global set everywhere
    tr = {0: 0, 1: 1000, 2: 4000, 3: 4500, 4: 6000, 5: 9000, 6: 12000,        # round 0: wait 3 us
          9: 12500, 10: 20500, 11: 20500, 12: 22000, 13: 25000, 14: 28000,      # round 1: wait 8 us
          40: 28100, 41: 28100, 42: 30000}
    d = decode_k2_trace(tr, 0, 4)
    assert d["complete"] and d["total"] == 30.0 and d["wait"] == pytest.approx(11.0) and d["work"] == pytest.approx(19.0)
    assert [r["role"] for r in d["rounds"]] == ["recv", "recv"] and d["rounds"][1]["select"] == pytest.approx(3.0)
    # rank 1: round-0 sender, then waits for the broadcast
    tr1 = {0: 0, 7: 2000, 8: 3500, 40: 25000, 41: 27000, 42: 29000}
    d1 = decode_k2_trace(tr1, 1, 4)
    assert d1["rounds"][0] == {"role": "send", "push": 2.0, "flag": 1.5} and d1["bcast_wait"] == pytest.approx(21.5)
    assert d1["wait"] == pytest.approx(21.5) and d1["put_back"] == 2.0
    # rank 2: receiver in round 0, compacts straight into rank 0's slot (flag stamp of round 1), then waits
    tr2 = {0: 0, 1: 500, 2: 2500, 3: 3000, 4: 4000, 5: 6000, 6: 8000, 16: 8500, 40: 20000, 41: 21000, 42: 22000}
    d2 = decode_k2_trace(tr2, 2, 4)
    assert d2["rounds"][0]["role"] == "recv" and d2["rounds"][1].get("sent") is None and d2["rounds"][1]["role"] == "send"
    assert d2["wait"] == pytest.approx(2.0 + 11.5)
    assert decode_k2_trace({0: 0, 1: 5}, 0, 2) == {"complete": False}


def test_queue_driven_allreducer_signals_done_once_per_iteration(monkeypatch):
    """The reference's thread protocol (allreducer.py:497-597): parameter names arrive through a queue in
    backward order, a merged group is reduced when its last name is there, and "DONE" is posted once,
    after ALL groups of the iteration, not after the first one."""
    import queue
    import threading
    from gtopkssgd_b200.parallel.allreducer import AllReducer
    monkeypatch.setattr(settings, "PIN_DENSITY", True)
    torch.manual_seed(0)
    net, _ = create_net(10, "mnistnet")
    q1, q2 = queue.Queue(), queue.Queue()
    ar = AllReducer(net.named_parameters(), compression=compressors["gtopk"], sparse=True, density=0.01,
                    msg_queue=q1, msg_queue2=q2, threshold=8000)
    assert len(ar.engines) >= 2
    reduced = []
    orig = ar.reduce_group
    monkeypatch.setattr(ar, "reduce_group", lambda gi: (reduced.append(gi), orig(gi))[1])
    t = threading.Thread(target=ar.run, daemon=True)
    t.start()
    names = [n for n, _ in net.named_parameters()][::-1]
    for it in range(2):
        ar.flat.grad.normal_()
        for i, n in enumerate(names):
            q1.put(n)
            if i < len(names) - 1:
                time.sleep(0.002)
                assert q2.empty(), "DONE before every group was reduced"
        assert q2.get(timeout=10) == "DONE"
        assert q2.empty() and len(reduced) == (it + 1) * len(ar.engines)
    q1.put("STOP")
    t.join(timeout=5)
    assert not t.is_alive()


def test_failed_exchange_seen_on_the_host_mirror_stops_the_next_iteration(monkeypatch):
    """The exchange kernel leaves a sticky status in its result words, which are mirrored to pinned
    host memory behind every exchange; pre_iteration() looks at the mirror without synchronising,
    tells err_handler and raises before anything of the next iteration is launched.  (The device
    side of this is tests/test_gpu_kernels.py::test_k2_bounded_wait_reports_timeout; here the mirror
    is a fake.)"""
    from gtopkssgd_b200.parallel.allreducer import GTopkTimeout
    monkeypatch.setattr(settings, "PIN_DENSITY", True)
    net, _ = create_net(10, "mnistnet")
    calls = []
    opt = torch.optim.SGD(net.parameters(), lr=0.1)
    d = DistributedOptimizer(opt, net.named_parameters(), compression=compressors["gtopk"], is_sparse=True,
                             density=0.01, err_handler=lambda n, r: calls.append((n, r)))

    class FakeRankCtx:
        def __init__(self):
            self.words = (0, 0)

        def failed_on_host_mirror(self):
            return self.words

    fake = FakeRankCtx()
    d._allreducer.engines[0].rank_ctx = fake
    d.zero_grad()                      # healthy mirror: nothing happens
    fake.words = (1, 212)              # "timeout waiting for a peer flag" at code location 212
    with pytest.raises(GTopkTimeout, match="peer flag"):
        d.zero_grad()
    assert calls == [(1, 0)]
    d._allreducer.engines[0].rank_ctx = None
    d.stop()
