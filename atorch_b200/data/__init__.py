from .data_utils import expand_batch_dim, get_sample_batch
from .elastic_dataset import ElasticDataset, ShardService, get_elastic_dataloader
from .preloader import GpuPreLoader
from .shm_context import ShmDataContext, ShmDataloader
from .unordered_dataloader import UnorderedDataLoader, UnshuffledBatchDataLoader
from .coworker_dataset import CoworkerDataset, build_coworker_dataloader
