"""Evaluation driver: benchmarks, backends, job fan-out, graders."""
from tah_b200.evaluate.datasets import load_combined_dataset
from tah_b200.evaluate.jobs import (allocate_gpus_and_run_jobs, combine_job_results, parse_data_range,
                                    run_single_job)

__all__ = ["allocate_gpus_and_run_jobs", "combine_job_results", "load_combined_dataset", "parse_data_range",
           "run_single_job"]
