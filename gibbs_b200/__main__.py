import sys

from .engine.cli import main

sys.exit(main())
