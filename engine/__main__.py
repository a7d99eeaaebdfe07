import sys

from prism_b200.cli import main

sys.exit(main())
