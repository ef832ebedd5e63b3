"""``python -m chibillm_b200``: the command line (see chibillm_b200/cli.py)."""
import sys

from .cli import main

sys.exit(main())
