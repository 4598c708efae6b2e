"""Drop-in name: ``import robocache`` resolves to the B200-native implementation, so call sites
written against the reference (robocache/python/robocache/__init__.py:483-493) run unchanged."""
from robogoat_b200 import *  # noqa: F401,F403
from robogoat_b200 import __all__, __version__  # noqa: F401
