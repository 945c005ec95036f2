"""`python -m socrates_b200` is `python -m socrates_b200.inference_paged`."""
import sys

from .inference_paged import main

sys.exit(main())
