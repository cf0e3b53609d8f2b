"""`python -m rllm_b200 ...` is the same command line as `bin/rllm`."""
import sys

from .cli import main

sys.exit(main())
