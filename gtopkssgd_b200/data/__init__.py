"""Data pipeline: synthetic workloads of the named shapes, CIFAR-10 / MNIST /
ImageNet-HDF5 / PTB / AN4 readers, samplers and CTC decoders."""
