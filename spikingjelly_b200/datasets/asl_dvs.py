"""ASL-DVS: 24 American-sign-language letters recorded with a DAVIS240c, 180 x 240, MATLAB ``.mat`` files with
``ts, x, y, pol`` (``spikingjelly/datasets/asl_dvs.py:21-242``)."""
import shutil
from pathlib import Path
from typing import Callable, Optional, Tuple

from torchvision.datasets.utils import extract_archive

from ..logger import logger
from . import utils
from .base import NeuromorphicDatasetFolder, convert_class_tree, extract_all

__all__ = ["ASLDVS"]


def _read_mat_save_to_np(mat_file, np_file):
    import scipy.io
    m = scipy.io.loadmat(str(mat_file))
    # the recordings are mirrored on both axes with respect to the other datasets
    utils.np_savez(str(np_file), t=m["ts"].squeeze(), x=239 - m["x"].squeeze(), y=179 - m["y"].squeeze(), p=m["pol"].squeeze())


class ASLDVS(NeuromorphicDatasetFolder):
    def __init__(self, root: str, data_type: str = "event", frames_number: int = None, split_by: str = None,
                 duration: int = None, custom_integrate_function: Callable = None,
                 custom_integrated_frames_dir_name: str = None, transform: Optional[Callable] = None,
                 target_transform: Optional[Callable] = None):
        super().__init__(root, None, data_type, frames_number, split_by, duration, custom_integrate_function,
                         custom_integrated_frames_dir_name, transform, target_transform)

    @classmethod
    def get_H_W(cls) -> Tuple:
        return 180, 240

    @classmethod
    def resource_url_md5(cls) -> list:
        logger.warning("ICCV2019_DVS_dataset.zip is re-packed by the file host, so its MD5 is not checked; if the link has "
                       "expired, fetch the OpenI mirror (`openi dataset download OpenI/ASLDVS`) and unpack ASLDVS.zip.")
        return [("ICCV2019_DVS_dataset.zip", "https://www.dropbox.com/sh/ibq0jsicatn7l6r/AACNrNELV56rs1YInMWUs9CAa?dl=0", None)]

    @classmethod
    def downloadable(cls) -> bool:
        return False

    @classmethod
    def extract_downloaded_files(cls, download_root: Path, extract_root: Path):
        tmp = download_root / "temp_ext"
        tmp.mkdir()
        extract_archive(download_root / "ICCV2019_DVS_dataset.zip", tmp)
        extract_all([z for z in tmp.iterdir() if z.suffix == ".zip"], extract_root, max_workers=2)
        shutil.rmtree(tmp)

    @classmethod
    def create_raw_from_extracted(cls, extract_root: Path, raw_root: Path):
        convert_class_tree(extract_root, raw_root, _read_mat_save_to_np)
