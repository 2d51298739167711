"""Same import name as the reference module: small host-side helpers."""
from gtopkssgd_b200.utils.misc import (autolabel, create_path, force_insert_item, gen_random_id, topk,  # noqa: F401
                                        update_fontsize)
