"""``galvatron.utils`` under its reference name (galvatron/utils/__init__.py:1-4)."""
from hetu_galvatron_b200.utils import *  # noqa: F401,F403
