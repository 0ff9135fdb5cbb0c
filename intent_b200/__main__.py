"""``python -m intent_b200 describe|doctor``: the backend's view of the reference's tool commands."""
import sys

from .tools import main

sys.exit(main())
