"""Same import name as the reference module: ``from compression import compressors``."""
from gtopkssgd_b200.parallel.compression import (NoneCompressor, TopKCompressor, TopKCompressor2,  # noqa: F401
                                                  compressors, gTopKCompressor)
