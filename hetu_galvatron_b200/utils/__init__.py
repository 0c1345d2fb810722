from .config_utils import (array2str, config2strategy, dict_join_dirname, num2str, read_allreduce_bandwidth_config,
                           read_json_config, read_p2p_bandwidth_config, remap_config, str2array, strategy2config,
                           write_json_config)
from .memory_utils import memory_stats_mb, print_peak_memory
from .strategy_utils import form_strategy, print_strategies, strategy_str2list
from .training_utils import distributed_dataloader, print_loss, set_seed
from .attr_utils import mixed_precision_dtype, print_param_num, rgetattr, rhasattr, rsetattr
