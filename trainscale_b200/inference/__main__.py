import sys

from .engine import main

sys.exit(main())
