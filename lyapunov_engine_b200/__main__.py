import sys

from .entrypoints.cli import main

sys.exit(main())
