"""``python -m glm_tpu_b200`` runs the command line (see ``entrypoints/cli/main.py``)."""

import sys

from glm_tpu_b200.entrypoints.cli.main import main

sys.exit(main())
