from .arguments import galvatron_search_args
from .cost_model import MemoryCostModel, OtherTimeCostModel, TimeCostModel, pipeline_costmodel
from .cost_model_args import ModelArgs, ParallelArgs, ProfileHardwareArgs, ProfileModelArgs, TrainArgs
from .dynamic_programming import DPAlg, DpOnModel
from .search_engine import GalvatronSearchEngine
from .context_parallel import search_with_context_parallel
