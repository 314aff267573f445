"""``python -m pmetal_b200.cli <command> ...``"""
import sys

from .main import main

sys.exit(main())
