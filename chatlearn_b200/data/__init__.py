from .data import (EpisodeReplayBuffer, ReplaySampleManager, RLHFDataLoader, StreamDataset,
                   read_data_path_list)
from .prompt_dataset import PromptPipeline, VLPromptPipeline
from .sampler import (EpisodeDataSampler, EpochPermutation, MultiDatasetSampler, RLHFSingleSampler,
                      SingleDataSampler)
