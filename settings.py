"""Same import name as the reference module: run-wide switches and the logger."""
from gtopkssgd_b200.settings import *  # noqa: F401,F403
from gtopkssgd_b200.settings import add_file_handler, formatter, hostname, logger  # noqa: F401
