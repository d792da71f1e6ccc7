// SPDX-License-Identifier: MIT
//
// blrun -- SPMD launcher: runs a python script as N ranks of one node (one per
// GPU) with the environment that barlink's process group and torchrun-style
// scripts expect, and with no Linux capabilities in the payload.
//
//   blrun [-n N] [-p PORT] script.py [args...]
//
//   N      ranks to start: -n, else BL_NPROC, else the number of entries in
//          BL_DEVICES, else 1
//   N = 1  the reference's model (tools/blrun.c:7-24 there): exec
//          python -m barlink_sm86_b200._bootstrap script, which brings the link
//          up for BL_DEVICES / BL_POOL_MB in single-process mode, then runs the
//          script
//   N > 1  forks N children, each exec'ing the same bootstrap with RANK,
//          LOCAL_RANK, WORLD_SIZE, MASTER_ADDR=127.0.0.1, MASTER_PORT, BL_PG_ID
//          and BL_SKIP_INIT=1 (ranks bring the link up themselves through
//          init_process_group); LOCAL_RANK follows BL_DEVICES when given.
//          The first child that fails takes the others down (by exact pid) and
//          its exit code is returned.
//
// The reference's launcher exists to hold CAP_SYS_ADMIN across bl_init and to
// drop it before user code runs.  Nothing here needs a capability (NVLink peer
// memory is plain CUDA), so the launcher only guarantees the second half: the
// payload starts with no_new_privs set, an empty ambient set and, when the
// kernel lets us, no effective capabilities even for uid 0 (BL_KEEP_CAPS=1
// skips this).  Python is $BL_PYTHON or `python3` from PATH.
#define _GNU_SOURCE
#include <errno.h>
#include <libgen.h>
#include <limits.h>
#include <signal.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/prctl.h>
#include <sys/syscall.h>
#include <sys/wait.h>
#include <unistd.h>

#ifndef SECBIT_NOROOT
#define SECBIT_NOROOT 0x01
#define SECBIT_NOROOT_LOCKED 0x02
#endif

static void drop_privileges(void) {
  if (getenv("BL_KEEP_CAPS") && getenv("BL_KEEP_CAPS")[0] == '1') return;
  prctl(PR_SET_NO_NEW_PRIVS, 1, 0, 0, 0);
  prctl(PR_CAP_AMBIENT, PR_CAP_AMBIENT_CLEAR_ALL, 0, 0, 0);
  // uid 0 would regain every capability at execve; NOROOT stops that (needs
  // CAP_SETPCAP, which an unprivileged user neither has nor needs)
  prctl(PR_SET_SECUREBITS, SECBIT_NOROOT | SECBIT_NOROOT_LOCKED, 0, 0, 0);
  struct {
    unsigned version;
    int pid;
  } hdr = {0x20080522u, 0};
  struct {
    unsigned effective, permitted, inheritable;
  } data[2];
  memset(data, 0, sizeof(data));
  syscall(SYS_capset, &hdr, data);
}

static int count_devices(const char* s) {
  if (!s || !*s) return 0;
  int n = 1;
  for (; *s; ++s)
    if (*s == ',') ++n;
  return n;
}

static int nth_device(const char* s, int i) {
  if (!s || !*s) return i;
  const char* p = s;
  for (int k = 0; k < i && p; ++k) {
    p = strchr(p, ',');
    if (p) ++p;
  }
  return p ? atoi(p) : i;
}

static void usage(void) {
  fprintf(stderr,
          "usage: blrun [-n N] [-p PORT] script.py [args...]\n"
          "env: BL_DEVICES=0,1,..  BL_POOL_MB=1024  BL_NPROC=N  BL_PYTHON=/path/to/python  BL_KEEP_CAPS=1\n");
}

int main(int argc, char** argv) {
  int nproc = 0, port = 0, ai = 1;
  while (ai < argc && argv[ai][0] == '-') {
    if (!strcmp(argv[ai], "-n") && ai + 1 < argc) {
      nproc = atoi(argv[ai + 1]);
      ai += 2;
    } else if (!strcmp(argv[ai], "-p") && ai + 1 < argc) {
      port = atoi(argv[ai + 1]);
      ai += 2;
    } else if (!strcmp(argv[ai], "--")) {
      ++ai;
      break;
    } else {
      usage();
      return 2;
    }
  }
  if (ai >= argc) {
    usage();
    return 2;
  }
  const char* devs = getenv("BL_DEVICES");
  if (nproc <= 0 && getenv("BL_NPROC")) nproc = atoi(getenv("BL_NPROC"));
  if (nproc <= 0) nproc = 1;
  if (nproc > 8) {
    fprintf(stderr, "blrun: at most 8 ranks per node (got %d)\n", nproc);
    return 2;
  }
  if (nproc > 1 && devs && count_devices(devs) < nproc) {
    fprintf(stderr, "blrun: BL_DEVICES lists %d GPUs but %d ranks were asked for\n", count_devices(devs),
            nproc);
    return 2;
  }

  // the repo root (for PYTHONPATH) is the parent of this executable's directory
  char self[PATH_MAX], repo[PATH_MAX];
  ssize_t n = readlink("/proc/self/exe", self, sizeof(self) - 1);
  if (n < 0) {
    perror("readlink(/proc/self/exe)");
    return 1;
  }
  self[n] = 0;
  strncpy(repo, self, sizeof(repo) - 1);
  repo[sizeof(repo) - 1] = 0;
  dirname(repo);
  dirname(repo);
  const char* old = getenv("PYTHONPATH");
  char pypath[PATH_MAX * 2];
  if (old && *old) snprintf(pypath, sizeof(pypath), "%s:%s", repo, old);
  else snprintf(pypath, sizeof(pypath), "%s", repo);
  setenv("PYTHONPATH", pypath, 1);
  const char* python = getenv("BL_PYTHON");
  if (!python || !*python) python = "python3";

  int extra = 3;
  char** nargv = calloc((size_t)(argc - ai) + extra + 1, sizeof(char*));
  if (!nargv) {
    perror("calloc");
    return 1;
  }
  nargv[0] = (char*)python;
  nargv[1] = (char*)"-m";
  nargv[2] = (char*)"barlink_sm86_b200._bootstrap";
  for (int i = ai; i < argc; ++i) nargv[i - ai + extra] = argv[i];

  drop_privileges();

  if (nproc == 1) {
    execvp(python, nargv);
    perror("blrun: exec python");
    return 1;
  }

  if (port <= 0) port = 20000 + (int)(getpid() % 20000);
  char buf[64];
  setenv("MASTER_ADDR", "127.0.0.1", 1);
  snprintf(buf, sizeof(buf), "%d", port);
  setenv("MASTER_PORT", buf, 1);
  snprintf(buf, sizeof(buf), "%d", nproc);
  setenv("WORLD_SIZE", buf, 1);
  setenv("LOCAL_WORLD_SIZE", buf, 1);
  setenv("BL_SKIP_INIT", "1", 1);
  snprintf(buf, sizeof(buf), "blrun%d", (int)getpid());
  setenv("BL_PG_ID", buf, 0);

  pid_t pids[8];
  for (int r = 0; r < nproc; ++r) {
    pid_t p = fork();
    if (p < 0) {
      perror("blrun: fork");
      for (int k = 0; k < r; ++k) kill(pids[k], SIGTERM);
      return 1;
    }
    if (p == 0) {
      snprintf(buf, sizeof(buf), "%d", r);
      setenv("RANK", buf, 1);
      snprintf(buf, sizeof(buf), "%d", nth_device(devs, r));
      setenv("LOCAL_RANK", buf, 1);
      execvp(python, nargv);
      perror("blrun: exec python");
      _exit(127);
    }
    pids[r] = p;
  }
  int rc = 0, left = nproc;
  while (left > 0) {
    int st = 0;
    pid_t p = wait(&st);
    if (p < 0) {
      if (errno == EINTR) continue;
      break;
    }
    --left;
    int code = WIFEXITED(st) ? WEXITSTATUS(st) : 128 + (WIFSIGNALED(st) ? WTERMSIG(st) : 0);
    for (int r = 0; r < nproc; ++r)
      if (pids[r] == p) pids[r] = -1;
    if (code != 0 && rc == 0) {
      rc = code;
      // a failed rank leaves the others waiting on it: stop exactly our children
      for (int r = 0; r < nproc; ++r)
        if (pids[r] > 0) kill(pids[r], SIGTERM);
    }
  }
  return rc;
}
