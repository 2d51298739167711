"""Text reports:  python -m gtopkssgd_b200.analysis.report [--log FILE] [--models]

--models  prints the alpha-beta predictions for dense / Top-k / gTop-k and the
          published scaling efficiencies;
--log     summarises a trainer log (epoch losses, validation metric, mean speed,
          communication profile);
--p2p     fits time = alpha + beta * size to a point-to-point probe log;
--allreduce-log FILE --workers N   compares a measured all-reduce log with the
          ring model (mean relative error);
--layers  per-layer log: message-size statistics and the WFBP / single /
          merged timeline totals."""
from __future__ import annotations

import argparse

from . import cost_models as cm
from .log_parser import mean_speed, parse_log


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--log", type=str, default=None)
    ap.add_argument("--models", action="store_true")
    ap.add_argument("--m", type=int, default=25 * 1024 * 1024)
    ap.add_argument("--rho", type=float, default=0.001)
    ap.add_argument("--p2p", type=str, default=None)
    ap.add_argument("--allreduce-log", type=str, default=None)
    ap.add_argument("--workers", type=int, default=4)
    ap.add_argument("--layers", type=str, default=None)
    args = ap.parse_args(argv)
    from . import comm_logs as cl
    if args.p2p:
        sizes, mean, _ = cl.read_allreduce_log(args.p2p)
        alpha, beta = cl.fit_alpha_beta(sizes, mean)
        print("point-to-point fit over %d sizes: alpha = %.6f, beta = %.9f per unit of size" % (len(sizes), alpha, beta))
    if args.allreduce_log:
        sizes, mean, _ = cl.read_allreduce_log(args.allreduce_log)
        pred = cl.predict_allreduce(sizes, args.workers)
        print("all-reduce on %d workers, %d sizes: mean relative error of the ring model %.3f"
              % (args.workers, len(sizes), cl.relative_error(mean, pred)))
    if args.layers:
        sizes, comms, computes, _ = cl.read_layer_log(args.layers)
        print("layers:", dict(cl.gradient_size_statistics(sizes)))
        sim = cm.Simulator(args.layers, computes, sizes, args.workers)
        print("iteration time [ms]: WFBP %.3f, single all-reduce %.3f, merged %.3f"
              % (sim.wfbp(comms).total_ms, sim.single_allreduce().total_ms, sim.mg_wfbp().total_ms))
    if args.models or not (args.log or args.p2p or args.allreduce_log or args.layers):
        print("all-reduce models, m=%d elements, rho=%g (ms, 1 GbE constants)" % (args.m, args.rho))
        print("%6s %12s %12s %12s" % ("P", "dense", "topk", "gtopk"))
        for p in (4, 8, 16, 32, 64, 128):
            print("%6d %12.2f %12.2f %12.2f" % (p, cm.dense_allreduce_ms(p, args.m),
                                                 cm.topk_allreduce_ms(p, args.m, args.rho),
                                                 cm.gtopk_allreduce_ms(p, args.m, args.rho)))
        for model, t in cm.PUBLISHED_THROUGHPUT.items():
            print(model, "gTop-k scaling efficiency %:", ["%.1f" % v for v in cm.scaling_efficiency(t["gtopk"])],
                  "vs dense:", ["%.2fx" % v for v in cm.speedup_over(t["gtopk"], t["dense"])])
    if args.log:
        log = parse_log(args.log)
        print("epochs:", len(log.epochs), "num_batches_per_epoch:", log.num_batches_per_epoch)
        for e, l, a in zip(log.epochs, log.train_loss, log.train_acc):
            print("  epoch %d loss %.4f acc %.3f" % (e, l, a))
        for e, l, a in zip(log.val_epochs, log.val_loss, log.val_acc):
            print("  val epoch %d loss %.4f metric %.4f" % (e, l, a))
        print("mean speed (images/s per worker):", mean_speed(log))
        for row in log.profiling[-3:]:
            print("  profile", row)


if __name__ == "__main__":
    main()
