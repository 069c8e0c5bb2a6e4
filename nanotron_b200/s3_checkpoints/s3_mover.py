"""Background checkpoint transfer to / from object storage through the ``s5cmd`` command-line tool
(parity: reference src/nanotron/s3_checkpoints/s3_mover.py).

A small state machine: IDLE -> UPLOADING -> (REMOVING_CHECKPOINT ->) IDLE, and IDLE -> DOWNLOADING -> IDLE.  The
transfer runs as a subprocess; ``update()`` is polled from the training loop.  A non-zero exit code is logged and the
mover returns to IDLE keeping the local files, so a failed upload never loses a checkpoint.  Only one process per
node does real work (``dummy=True`` elsewhere); ``distributed_wait_for_completion`` lets all ranks agree that every
node has finished.
"""
from __future__ import annotations

import glob
import json
import os
import subprocess
import time
from datetime import datetime
from enum import Enum
from typing import Optional, Union

import torch
from filelock import FileLock, Timeout

from nanotron_b200 import distributed as dist
from nanotron_b200 import logging
from nanotron_b200.logging import human_format, log_rank

logger = logging.get_logger(__name__)


class S3Mover:
    class S3MoverState(Enum):
        IDLE = "IDLE"
        UPLOADING = "UPLOADING"
        DOWNLOADING = "DOWNLOADING"
        REMOVING_CHECKPOINT = "REMOVING_CHECKPOINT"

    class DummyPopen:
        def __init__(self, *args, **kwargs):
            pass

        def poll(self):
            return 0

        def communicate(self):
            return ("", "")

    def __init__(self, local_path, s3_path, post_upload_callback=None, remove_after_upload: Optional[bool] = True, s5cmd_numworkers: Optional[int] = None, s5cmd_concurrency: Optional[int] = None, s5cmd_path: Optional[str] = None, s5cmd_credentials: Optional[str] = None, clean_up_local_on_start: bool = False, dummy: bool = False, s3_region: str = "us-east-1"):
        self.process: Optional[Union[subprocess.Popen, S3Mover.DummyPopen]] = None
        self.remove_after_upload = remove_after_upload
        self.s5cmd_numworkers = s5cmd_numworkers
        self.s5cmd_concurrency = s5cmd_concurrency
        self.s5cmd_path = str(s5cmd_path) if s5cmd_path is not None else "s5cmd"
        self.s5cmd_credentials = s5cmd_credentials
        self.lock_file = None
        self.dummy = dummy
        self.s3_region = s3_region
        self.post_upload_callback = post_upload_callback
        self.post_upload_callback_outputs = None
        local_path, s3_path = str(local_path), str(s3_path)
        self.local_path = local_path if local_path.endswith("/") else local_path + "/"
        self.s3_path = s3_path if s3_path.endswith("/") else s3_path + "/"
        self.s3_path_direct_link = f"https://s3.console.aws.amazon.com/s3/buckets/{self.s3_path[5:]}?region={self.s3_region}"
        self._reset_state()
        if clean_up_local_on_start:
            self._start_removing()

    def _warning(self, message):
        log_rank(message, logger=logger, level=logging.WARNING)

    def _info(self, message):
        log_rank(message, logger=logger, level=logging.INFO)

    def _reset_state(self):
        self.state = self.S3MoverState.IDLE
        self.num_uploaded_files = 0
        if self.lock_file is not None:
            self._release_lock()
        self.lock_file = None
        self.stdout = ""
        self.start_time: Optional[datetime] = None
        self.cmd = ""

    def _popen(self, cmd: list):
        self.stdout = ""
        self.start_time = datetime.now()
        self.cmd = cmd
        if self.dummy:
            return self.DummyPopen(cmd)
        try:
            process = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
            os.set_blocking(process.stdout.fileno(), False)
            return process
        except FileNotFoundError as e:
            self._warning(f"Could not start {cmd[0]}: {e}")
            failed = self.DummyPopen()
            failed.poll = lambda: 127
            return failed

    def _acquire_lock(self, file_path: str) -> bool:
        if self.dummy:
            return True
        if file_path.endswith("/"):
            lock_file_path = file_path[:-1] + ".lock"
        else:
            lock_file_path = file_path + ".lock"
        self.lock_file = FileLock(lock_file_path)
        try:
            self.lock_file.acquire(timeout=1)
        except Timeout:
            self._warning(f"S3Mover: Could not acquire lock {lock_file_path}; another process is working on it")
            return False
        return True

    def _release_lock(self):
        if self.dummy or self.lock_file is None:
            return
        if self.lock_file.is_locked:
            self.lock_file.release()

    def get_state_as_int(self) -> int:
        """0 when idle, 1 while a transfer or removal is in flight."""
        return 0 if self.state == self.S3MoverState.IDLE else 1

    def get_current_stdout(self) -> str:
        if self.process is None or isinstance(self.process, self.DummyPopen):
            return ""
        try:
            out = self.process.stdout.read()
        except (ValueError, OSError):
            out = None
        if out:
            self.stdout += out.decode(errors="replace")
        return self.stdout

    def wait_for_completion(self):
        while self.state != self.S3MoverState.IDLE:
            self.update()
            time.sleep(0.5)

    def distributed_wait_for_completion(self, group: Optional[dist.ProcessGroup] = None):
        """Block until every rank of ``group`` reports an idle mover."""
        if group is None or not dist.is_initialized():
            return self.wait_for_completion()
        device = torch.device("cuda") if dist.get_backend(group) == "nccl" else torch.device("cpu")
        while True:
            self.update()
            flag = torch.tensor([self.get_state_as_int()], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
            if int(flag.item()) == 0:
                break
            time.sleep(1)
        dist.barrier(group)

    def is_previous_save_finished(self) -> bool:
        self.update()
        return self.state == self.S3MoverState.IDLE

    # ---- transitions
    def start_uploading(self, sub_folder=None):
        self.update()
        if self.state != self.S3MoverState.IDLE:
            self._warning("S3Mover: upload requested while the previous transfer is not finished: skipping")
            return False
        local_path, s3_path = self.local_path, self.s3_path
        if sub_folder is not None:
            local_path, s3_path = os.path.join(local_path, sub_folder), os.path.join(s3_path, sub_folder)
        if not self._acquire_lock(local_path):
            return False
        self.state = self.S3MoverState.UPLOADING
        cmd = [self.s5cmd_path, "--json"]
        if self.s5cmd_credentials is not None:
            cmd += ["--credentials-file", self.s5cmd_credentials]
        if self.s5cmd_numworkers is not None:
            cmd += ["--numworkers", str(self.s5cmd_numworkers)]
        cmd += ["cp"]
        if self.s5cmd_concurrency is not None:
            cmd += ["--concurrency", str(self.s5cmd_concurrency)]
        cmd += ["--exclude", "*.lock", "--exclude", "*.lock.*", local_path, s3_path]
        self._info(f"S3Mover: start uploading {local_path} to {s3_path}")
        self.process = self._popen(cmd)
        return True

    def start_downloading(self):
        self.update()
        if self.state != self.S3MoverState.IDLE:
            return False
        if not self._acquire_lock(self.local_path):
            return False
        self.state = self.S3MoverState.DOWNLOADING
        cmd = [self.s5cmd_path, "--json"]
        if self.s5cmd_credentials is not None:
            cmd += ["--credentials-file", self.s5cmd_credentials]
        if self.s5cmd_numworkers is not None:
            cmd += ["--numworkers", str(self.s5cmd_numworkers)]
        cmd += ["cp"]
        if self.s5cmd_concurrency is not None:
            cmd += ["--concurrency", str(self.s5cmd_concurrency)]
        cmd += [self.s3_path + "*", self.local_path]
        self._info(f"S3Mover: start downloading {self.s3_path} to {self.local_path}")
        self.process = self._popen(cmd)
        return True

    def _start_removing(self):
        self.state = self.S3MoverState.REMOVING_CHECKPOINT
        top = [d for d in glob.glob(self.local_path + "*") if os.path.isdir(d)]
        self._info(f"S3Mover: removing local checkpoint folders {top}")
        self.process = self._popen(["rm", "-rf"] + top) if top else self.DummyPopen()

    def update(self) -> "S3Mover.S3MoverState":
        """Advance the state machine; call regularly."""
        if self.process is None:
            self._reset_state()
            return self.state
        return_code = self.process.poll()
        if return_code is None:
            return self.state  # still running
        self.get_current_stdout()
        if return_code != 0:
            self._warning(f"S3Mover: {self.state.value} failed (exit code {return_code}) cmd={self.cmd}\n{self.stdout[-2000:]}")
            self.process = None
            self._reset_state()
            return self.state
        if self.state == self.S3MoverState.DOWNLOADING:
            self._info(f"S3Mover: download finished in {datetime.now() - self.start_time}")
            self.process = None
            self._reset_state()
        elif self.state == self.S3MoverState.UPLOADING:
            total_files, total_size = 0, 0
            for line in self.stdout.splitlines():
                try:
                    rec = json.loads(line)
                    if rec.get("success"):
                        total_files += 1
                        total_size += int(rec.get("object", {}).get("size", 0))
                except (json.JSONDecodeError, AttributeError):
                    continue
            self.num_uploaded_files = total_files
            self._info(f"S3Mover: uploaded {total_files} files ({human_format(total_size)}B) in {datetime.now() - self.start_time} to {self.s3_path_direct_link}")
            if self.post_upload_callback is not None:
                self.post_upload_callback_outputs = self.post_upload_callback(uploaded_files=self.stdout)
            self.process = None
            self._release_lock()
            if self.remove_after_upload:
                self._start_removing()
            else:
                self._reset_state()
        elif self.state == self.S3MoverState.REMOVING_CHECKPOINT:
            self.process = None
            self._reset_state()
        return self.state
