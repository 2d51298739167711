"""Training drivers: trainer core, gTop-k / dense / single-GPU command lines,
and the checkpoint evaluator."""
