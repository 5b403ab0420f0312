"""``python -m skyrl_isoexec_b200.debug TRACE_A TRACE_B`` (stdlib-only entry point)."""
import sys

from .compare import main

sys.exit(main())
