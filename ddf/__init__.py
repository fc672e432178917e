"""Import-path alias so code written against the reference keeps working:
``from ddf import ddf, DDFPack`` (as in the reference's ddf_resnet.py:7,
test_time.py:8 and grad_check.py:8) resolves to ddfnet_b200."""
from ddfnet_b200 import *  # noqa: F401,F403
from ddfnet_b200 import __all__  # noqa: F401
