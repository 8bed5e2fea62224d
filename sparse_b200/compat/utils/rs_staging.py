"""`utils.rs_staging` of the reference (utils/rs_staging.py:11-118) under its
own names, over `sparse_b200.staging`."""
from sparse_b200.staging import DemandView as DemandCacheView  # noqa: F401
from sparse_b200.staging import StagingJob as TargetJob  # noqa: F401
from sparse_b200.staging import Transfer, select_candidates  # noqa: F401
