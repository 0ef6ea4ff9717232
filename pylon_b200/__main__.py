import sys

from pylon_b200.main import main

sys.exit(main())
