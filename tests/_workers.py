"""Rank functions used by the multi-process tests (imported by name in the
spawned children)."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402


def _make_batch(rank, it, bs):
    g = torch.Generator().manual_seed(1000 * it + rank)
    return torch.randn(bs, 3, 32, 32, generator=g), torch.randint(0, 10, (bs,), generator=g)


def resnet20_gtopk_worker(rank, world, iters, density, compressor, device_kind="cpu", threshold=None):
    """Plumbing configuration: ResNet-20; batch 32 per worker would be slow on CPU,
    batch 8 keeps the same code path.  Returns the final flat parameters."""
    from gtopkssgd_b200 import settings
    from gtopkssgd_b200.models import create_net
    from gtopkssgd_b200.parallel import comm
    from gtopkssgd_b200.parallel.compression import compressors
    from gtopkssgd_b200.parallel.distributed_optimizer import DistributedOptimizer
    settings.PIN_DENSITY = True
    settings.TRANSPORT = os.environ.get("GTOPK_TRANSPORT", settings.TRANSPORT)
    settings.logger.setLevel("WARNING")
    torch.set_num_threads(1)
    dev = torch.device("cpu")
    if device_kind == "cuda":
        dev = torch.device("cuda", rank)
        torch.cuda.set_device(dev)
    comm.init(backend="gloo" if device_kind == "cpu" else "nccl")
    torch.manual_seed(0)
    net, _ = create_net(10, "resnet20")
    net.to(dev)
    comm.broadcast_parameters(net.state_dict(), 0)
    opt = torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
    sparse = compressor != "none"
    dopt = DistributedOptimizer(opt, net.named_parameters(), compression=compressors[compressor], is_sparse=sparse,
                                density=density, wait_limit_ms=20000, threshold=threshold)
    crit = torch.nn.CrossEntropyLoss()
    fb = dopt._flat
    trace = {"p0": fb.param.detach().cpu().clone(), "grads": [], "params": [], "resid": [],
             "groups": [(g.start, g.numel, g.param_numel) for g in fb.groups]}
    for it in range(iters):
        x, y = _make_batch(rank, it, 8)
        dopt.zero_grad()
        crit(net(x.to(dev)), y.to(dev)).backward()
        if compressor == "none":
            dopt.synchronize()  # the in-place all-reduce must be complete before the buffer is recorded
        trace["grads"].append(fb.grad.detach().cpu().clone())  # raw local gradient (selection does not modify it)
        dopt.step()
        trace["params"].append(fb.param.detach().cpu().clone())
        trace["resid"].append(fb.residual.detach().cpu().clone())
    if device_kind == "cuda":
        torch.cuda.synchronize()
        dopt.check_status()
    trace["numel"] = fb.numel
    dopt.stop()
    comm.shutdown()
    return trace


def graphed_step_worker(rank, world, iters, compressor):
    """Whole-iteration CUDA graph (3 eager warm-up iterations, then replays)
    with a learning rate that changes between replays."""
    from gtopkssgd_b200 import settings
    from gtopkssgd_b200.parallel import comm
    from gtopkssgd_b200.parallel.compression import compressors
    from gtopkssgd_b200.parallel.distributed_optimizer import DistributedOptimizer
    from gtopkssgd_b200.trainer.dl_trainer import DLTrainer
    from gtopkssgd_b200.trainer.graphed_step import GraphedStep
    settings.PIN_DENSITY = True
    settings.logger.setLevel("WARNING")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    comm.init(backend="nccl")
    torch.manual_seed(0)
    t = DLTrainer(rank, world, dist=False, ngpus=1, batch_size=8, data_dir="synthetic", dataset="cifar10",
                  dnn="resnet20", lr=0.1, nworkers=world, device=dev, synthetic_train_size=256)
    comm.broadcast_parameters(t.net.state_dict(), 0)
    dopt = DistributedOptimizer(t.optimizer, t.net.named_parameters(), compression=compressors[compressor],
                                is_sparse=compressor != "none", density=0.001, wait_limit_ms=20000)
    t.update_optimizer(dopt)
    fb = dopt._flat
    step = GraphedStep(t, warmup=3)
    trace = {"p0": fb.param.detach().cpu().clone(), "grads": [], "params": [], "resid": [], "lrs": [],
             "numel": fb.numel, "groups": [(g.start, g.numel, g.param_numel) for g in fb.groups]}
    for it in range(iters):
        x, y = _make_batch(rank, it, 8)
        lr = 0.1 if it < 4 else 0.05
        for pg in dopt.param_groups:
            pg["lr"] = lr
        step.run(x.to(dev), y.to(dev))
        torch.cuda.synchronize()
        trace["lrs"].append(lr)
        trace["grads"].append(fb.grad.detach().cpu().clone())
        trace["params"].append(fb.param.detach().cpu().clone())
        trace["resid"].append(fb.residual.detach().cpu().clone())
    dopt.check_status()
    trace["graphs"] = len(step.graphs)
    dopt.stop()
    comm.shutdown()
    return trace


def leaving_peer_worker(rank, world):
    """Rank 1 leaves in an orderly way after one iteration; rank 0 must learn
    of it on the host before launching anything of the next iteration."""
    import time
    from gtopkssgd_b200 import settings
    from gtopkssgd_b200.models import create_net
    from gtopkssgd_b200.parallel import comm
    from gtopkssgd_b200.parallel.allreducer import GTopkTimeout
    from gtopkssgd_b200.parallel.compression import compressors
    from gtopkssgd_b200.parallel.distributed_optimizer import DistributedOptimizer
    settings.PIN_DENSITY = True
    settings.logger.setLevel("CRITICAL")
    torch.set_num_threads(1)
    comm.init(backend="gloo", timeout_s=30)
    torch.manual_seed(0)
    net, _ = create_net(10, "resnet20")
    calls = []
    opt = torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.9)
    dopt = DistributedOptimizer(opt, net.named_parameters(), compression=compressors["gtopk"], is_sparse=True,
                                density=0.001, err_handler=lambda n, r: calls.append((n, r)), wait_limit_ms=30000,
                                membership_check_every=1)
    crit = torch.nn.CrossEntropyLoss()
    x, y = _make_batch(rank, 0, 4)
    dopt.zero_grad()
    crit(net(x), y).backward()
    dopt.step()
    if rank == 1:
        dopt.stop()  # announces the departure
        time.sleep(3.0)  # keep the store reachable while rank 0 looks
        return "left"
    time.sleep(1.0)
    t0 = time.time()
    try:
        dopt.zero_grad()
        return "no error"
    except GTopkTimeout as exc:
        return ("left-detected", round(time.time() - t0, 2), calls, str(exc))


def failing_peer_worker(rank, world, mode):
    """Fault injection on the host: rank 1 leaves (or stalls) before the
    exchange; rank 0 must get a PeerTimeout / err_handler call, not a hang."""
    import time
    from gtopkssgd_b200 import settings
    from gtopkssgd_b200.models import create_net
    from gtopkssgd_b200.parallel import comm
    from gtopkssgd_b200.parallel.allreducer import GTopkTimeout
    from gtopkssgd_b200.parallel.compression import compressors
    from gtopkssgd_b200.parallel.distributed_optimizer import DistributedOptimizer
    settings.PIN_DENSITY = True
    settings.logger.setLevel("CRITICAL")
    torch.set_num_threads(1)
    comm.init(backend="gloo", timeout_s=30)
    torch.manual_seed(0)
    net, _ = create_net(10, "resnet20")
    calls = []
    opt = torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.9)
    dopt = DistributedOptimizer(opt, net.named_parameters(), compression=compressors["gtopk"], is_sparse=True,
                                density=0.001, err_handler=lambda n, r: calls.append((n, r)), wait_limit_ms=3000)
    crit = torch.nn.CrossEntropyLoss()
    x, y = _make_batch(rank, 0, 4)
    # start the good iteration together: the short wait limit is meant for the missing peer of the second
    # iteration, not for the start-up skew between two processes on a busy host
    torch.distributed.barrier()
    dopt.zero_grad()
    crit(net(x), y).backward()
    dopt.step()  # one good iteration with both ranks
    if rank == 1:
        if mode == "exit":
            os._exit(0)  # leaves between steps, nothing in flight
        if mode == "stall":
            time.sleep(9.0)  # three times rank 0's wait limit
            return "stalled"
    dopt.zero_grad()
    t0 = time.time()
    try:
        crit(net(x), y).backward()  # on CPU the group is reduced inside the last gradient hook
        dopt.step()
        return "no error"
    except GTopkTimeout:
        return ("timeout", round(time.time() - t0, 1), calls)


def interrupted_trainer_worker(rank, world, workdir):
    """The gTop-k training driver on two gloo ranks; rank 1 finishes after two
    iterations (an orderly departure), rank 0 wants ten.  Rank 0 must stop
    with GTopkTimeout before launching its third iteration and leave the state
    of iteration 2 on disk."""
    import glob
    import time
    from gtopkssgd_b200 import settings
    from gtopkssgd_b200.parallel import comm
    from gtopkssgd_b200.parallel.allreducer import GTopkTimeout
    from gtopkssgd_b200.trainer import gtopk_trainer
    from gtopkssgd_b200.trainer.dl_trainer import DLTrainer
    os.makedirs(os.path.join(workdir, str(rank)), exist_ok=True)
    os.chdir(os.path.join(workdir, str(rank)))
    settings.PIN_DENSITY = True
    settings.logger.setLevel("CRITICAL")
    torch.set_num_threads(1)
    comm.init(backend="gloo", timeout_s=30)
    if rank == 0:
        orig = DLTrainer.train_step

        def slow(self, *a, **k):
            if self.train_iter == 2:
                time.sleep(2.5)  # rank 1 has announced its departure by now
            return orig(self, *a, **k)

        DLTrainer.train_step = slow
    args = dict(dnn="mnistnet", dataset="mnist", data_dir="synthetic", nworkers=world, lr=0.01, batch_size=4,
                nsteps_update=1, max_epochs=1, compression=True, compressor="gtopk", density=0.01,
                max_iters=2 if rank == 1 else 10, membership_check_every=1)
    try:
        gtopk_trainer.robust_ssgd(**args)
    except GTopkTimeout as exc:
        files = glob.glob(os.path.join("weights", "**", "*-interrupted.pth"), recursive=True)
        ck = torch.load(files[0], map_location="cpu", weights_only=False) if files else {}
        return {"error": str(exc), "files": files, "iter": ck.get("iter"),
                "keys": sorted(ck.keys()), "n_resid": len(ck.get("residuals", {}))}
    if rank == 1:
        time.sleep(4.0)  # keep this process (and its connections) alive while rank 0 looks at the store
    return {"finished": True}


def flat_allreduce_worker(rank, world):
    from gtopkssgd_b200.parallel import comm
    from gtopkssgd_b200.parallel import flat_allreduce as fa
    torch.set_num_threads(1)
    comm.init(backend="gloo", timeout_s=30)
    torch.manual_seed(rank)  # different initial weights per rank: the wrapper must broadcast rank 0's
    net = torch.nn.Sequential(torch.nn.Linear(6, 4), torch.nn.ReLU(), torch.nn.Linear(4, 2))
    ddp = fa.DistributedDataParallel(net)
    w0 = torch.cat([p.detach().flatten() for p in net.parameters()]).clone()
    xs = [torch.full((3, 6), float(r + 1)) for r in range(world)]
    ddp(xs[rank]).sum().backward()
    fa.allreduce_gradients(net)
    grad = torch.cat([p.grad.flatten() for p in net.parameters()]).clone()
    # expected: mean over ranks of the local gradients, recomputed locally
    acc = None
    for r in range(world):
        net.zero_grad()
        net(xs[r]).sum().backward()
        g = torch.cat([p.grad.flatten() for p in net.parameters()])
        acc = g.clone() if acc is None else acc + g
    comm.shutdown()
    return {"grad": grad, "w0": w0, "expected": acc / world}


def gtopk_world3_worker(rank, world):
    from gtopkssgd_b200.models import create_net
    from gtopkssgd_b200.parallel import comm
    from gtopkssgd_b200.parallel.compression import compressors
    from gtopkssgd_b200.parallel.distributed_optimizer import DistributedOptimizer
    torch.set_num_threads(1)
    comm.init(backend="gloo", timeout_s=30)
    net, _ = create_net(10, "mnistnet")
    opt = torch.optim.SGD(net.parameters(), lr=0.1)
    try:
        DistributedOptimizer(opt, net.named_parameters(), compression=compressors["gtopk"], is_sparse=True)
        msg = "accepted"
    except ValueError as exc:
        msg = str(exc)
    comm.shutdown()
    return msg


def elastic_worker(rank, world, compressor, leaver, leave_iter, total_iters, device_kind="cpu"):
    """``leaver`` asks to leave at iteration ``leave_iter``; it trains up to the
    agreed iteration and returns, the others re-form a smaller job at that
    iteration and go on to ``total_iters``.  Every rank returns its history."""
    from gtopkssgd_b200 import settings
    from gtopkssgd_b200.models import create_net
    from gtopkssgd_b200.parallel import comm
    from gtopkssgd_b200.parallel.compression import compressors
    from gtopkssgd_b200.parallel.distributed_optimizer import DistributedOptimizer
    settings.PIN_DENSITY = True
    settings.logger.setLevel("ERROR")
    torch.set_num_threads(1)
    dev = torch.device("cpu")
    if device_kind == "cuda":
        dev = torch.device("cuda", rank)
        torch.cuda.set_device(dev)
    comm.init(backend="gloo" if device_kind == "cpu" else "nccl", timeout_s=60)
    torch.manual_seed(0)
    net, _ = create_net(10, "mnistnet")
    net.to(dev)
    net.eval()
    comm.broadcast_parameters(net.state_dict(), 0)
    calls = []
    opt = torch.optim.SGD(net.parameters(), lr=0.05, momentum=0.9)
    dopt = DistributedOptimizer(opt, net.named_parameters(), compression=compressors[compressor], is_sparse=True,
                                density=0.01, err_handler=lambda n, r: calls.append((n, r)), wait_limit_ms=30000,
                                membership_check_every=2, elastic=True)
    crit = torch.nn.CrossEntropyLoss()
    hist = []
    it = 0
    while it < total_iters:
        if rank == leaver and it == leave_iter:
            dopt.request_leave()
        if dopt.should_exit():
            break
        g = torch.Generator().manual_seed(100 * it + rank)
        x, y = torch.randn(4, 1, 28, 28, generator=g).to(dev), torch.randint(0, 10, (4,), generator=g).to(dev)
        dopt.zero_grad()
        crit(net(x), y).backward()
        dopt.step()
        hist.append((it, comm.size(), comm.rank(), dopt._allreducer.mode))
        it += 1
    if device_kind == "cuda":
        torch.cuda.synchronize()
        dopt.check_status()
    params = torch.cat([p.detach().flatten() for p in net.parameters()]).cpu().clone()
    out = {"hist": hist, "calls": calls, "params": params, "left_at": dopt.leave_at, "iters": it}
    dopt.stop()
    comm.shutdown()
    return out


def elastic_trainer_worker(rank, world, workdir):
    """The gTop-k training driver with --elastic semantics: rank 1 is asked to
    leave after two iterations; rank 0 must finish its ten iterations alone."""
    from gtopkssgd_b200 import settings
    from gtopkssgd_b200.parallel import comm
    from gtopkssgd_b200.trainer import gtopk_trainer
    os.makedirs(os.path.join(workdir, str(rank)), exist_ok=True)
    os.chdir(os.path.join(workdir, str(rank)))
    settings.PIN_DENSITY = True
    settings.logger.setLevel("CRITICAL")
    torch.set_num_threads(1)
    comm.init(backend="gloo", timeout_s=60)
    seen = {"n": 0}

    def asked():
        seen["n"] += 1
        return rank == 1 and seen["n"] >= 2

    trainer = gtopk_trainer.robust_ssgd(dnn="mnistnet", dataset="mnist", data_dir="synthetic", nworkers=world, lr=0.01,
                                        batch_size=4, nsteps_update=1, max_epochs=1, compression=True,
                                        compressor="gtopk", density=0.01, max_iters=10, membership_check_every=2,
                                        elastic=True, leave_requested=asked)
    out = {"iters": trainer.get_train_iter(), "nworkers": trainer.nworkers, "world_now": comm.size(),
           "loss": trainer.loss}
    comm.shutdown()
    return out


def slow_validation_worker(rank, world, workdir):
    """Epoch boundary with a validation pass on rank 0 that outlasts the exchange's
    wait limit: the other rank must wait for it on the host and training goes on."""
    import time
    from gtopkssgd_b200 import settings
    from gtopkssgd_b200.parallel import comm
    from gtopkssgd_b200.trainer import gtopk_trainer
    from gtopkssgd_b200.trainer.dl_trainer import DLTrainer
    os.makedirs(os.path.join(workdir, str(rank)), exist_ok=True)
    os.chdir(os.path.join(workdir, str(rank)))
    settings.PIN_DENSITY = True
    settings.WAIT_LIMIT_MS = 1500
    settings.logger.setLevel("CRITICAL")
    torch.set_num_threads(1)
    comm.init(backend="gloo", timeout_s=60)
    slept = {"n": 0}
    if rank == 0:
        def slow_test(self, epoch):
            slept["n"] += 1
            time.sleep(4.0)  # far longer than the 1.5 s exchange limit
            return 0.0
        DLTrainer.test = slow_test
    trainer = gtopk_trainer.robust_ssgd(dnn="mnistnet", dataset="mnist", data_dir="synthetic", nworkers=world, lr=0.01,
                                        batch_size=4, nsteps_update=1, max_epochs=3, compression=True,
                                        compressor="gtopk", density=0.01, max_iters=None, membership_check_every=1,
                                        synthetic_train_size=24)
    out = {"iters": trainer.get_train_iter(), "epoch": trainer.get_train_epoch(), "validations": slept["n"]}
    comm.shutdown()
    return out


def selfcheck_worker(rank, world, compressor):
    """Two training iterations on gloo ranks, then the checked exchange that bench.py
    runs at its end on real GPUs."""
    from gtopkssgd_b200 import settings
    from gtopkssgd_b200.models import create_net
    from gtopkssgd_b200.parallel import comm
    from gtopkssgd_b200.parallel.compression import compressors
    from gtopkssgd_b200.parallel.distributed_optimizer import DistributedOptimizer
    from gtopkssgd_b200.parallel.selfcheck import exchange_selfcheck
    settings.PIN_DENSITY = True
    settings.logger.setLevel("ERROR")
    torch.set_num_threads(1)
    comm.init(backend="gloo", timeout_s=60)
    torch.manual_seed(0)
    net, _ = create_net(10, "mnistnet")
    comm.broadcast_parameters(net.state_dict(), 0)
    opt = torch.optim.SGD(net.parameters(), lr=0.05, momentum=0.9)
    dopt = DistributedOptimizer(opt, net.named_parameters(), compression=compressors[compressor], is_sparse=True,
                                density=0.01, wait_limit_ms=30000, threshold=8000)
    crit = torch.nn.CrossEntropyLoss()
    for it in range(2):
        g = torch.Generator().manual_seed(100 * it + rank)
        x, y = torch.randn(4, 1, 28, 28, generator=g), torch.randint(0, 10, (4,), generator=g)
        dopt.zero_grad()
        crit(net(x), y).backward()
        dopt.step()
    dopt.zero_grad()
    crit(net(x), y).backward()  # leaves a fresh local gradient in the buffers, already reduced once by the hooks
    out = exchange_selfcheck(dopt)
    dopt.stop()
    comm.shutdown()
    return out


def fp16_wire_worker(rank, world):
    """Top-k all-gather with half-precision values on the wire (reference: allreducer.py:19-24, 52-53)."""
    import numpy as np
    from gtopkssgd_b200.parallel import comm, compat
    torch.set_num_threads(1)
    comm.init(backend="gloo", timeout_s=30)
    idx = np.arange(4, dtype=np.int64) + 10 * rank
    val = (np.arange(4, dtype=np.float32) + 1.0) * (1.0 + rank) / 3.0
    v, i, _ = compat.topk_sparse_allreduce(comm.cpu_group(), val, {}, indexes=idx, dtype=np.float16)
    comm.shutdown()
    return {"v": v, "i": i}


def real_peer_exchange_worker(rank, world, d, k, nctas, epochs, mode="gtopk"):
    """K1 + the exchange kernel between real GPUs (one process per GPU, CUDA-IPC symmetric regions),
    without a model around it: returns, per epoch, this rank's gradient seed, its local selection,
    the global result it holds and its residual, for the oracle comparison in the parent."""
    from gtopkssgd_b200 import settings
    from gtopkssgd_b200.ops import exchange as ex
    from gtopkssgd_b200.ops.select import TopkSelector, pairs_to_tensors
    from gtopkssgd_b200.parallel import comm
    settings.logger.setLevel("ERROR")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    comm.init(backend="nccl", timeout_s=120)
    with_ag = mode != "gtopk"
    region = ex.SymmetricRegion.create_ipc(ex.region_bytes(k, with_ag), group=comm.cpu_group())
    sel = TopkSelector(d, k, dev)
    resid = torch.zeros(d, device=dev)
    rc = ex.ExchangeRank(rank, world, d, k, sel, resid, region, with_allgather=with_ag, reselect=(mode == "topk2"))
    out = {"epochs": []}
    for e in range(epochs):
        g = torch.Generator(device=dev).manual_seed(1000 * e + rank)
        grad = torch.randn(d, device=dev, generator=g)
        sel.select(grad, resid, k)
        if mode == "gtopk":
            ex.launch_gtopk([rc], rc.desc, rank, world, k, nctas=nctas, limit_ms=10000)
        else:
            ex.launch_allgather([rc], rc.desc, rc.seg_counts, rank, world, k, reselect=(mode == "topk2"), nctas=nctas,
                                limit_ms=10000)
        torch.cuda.synchronize()
        li, lv = sel.pairs()
        n = int(rc.n_global.item())
        gout = ex.pairs_view(rc.gout_ptr(rc.last_parity()), n, dev)
        gi, gv = pairs_to_tensors(gout, n)
        out["epochs"].append({"local": (li.cpu(), lv.cpu()), "global": (gi.cpu(), gv.cpu()), "status": rc.status(),
                              "resid_sum": float(resid.double().sum()), "resid": resid.cpu().clone() if d <= 2_000_000 else None,
                              "guards": region.guards_intact()})
    comm.barrier()
    torch.cuda.synchronize()
    region.close()
    comm.shutdown()
    return out
