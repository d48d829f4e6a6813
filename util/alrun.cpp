// alrun - minimal single-host launcher: forks N copies of a program with the
// rank environment the library's bootstrap understands.
//
//   alrun -n 4 [--timeout SECONDS] [--nodes K] program [args...]
//
// Each child gets AL_RANK, AL_WORLD_SIZE, AL_LOCAL_RANK and a fresh AL_JOB_KEY.
// --nodes K models K nodes on this machine: consecutive blocks of N/K ranks get
// the same AL_NODE_ID, the TCP transport is selected and a free rendezvous port
// is chosen, so ranks of different blocks talk over loopback TCP and cannot
// share memory or pass descriptors - what ranks on different hosts see.
// If a child fails or the time limit passes, the remaining children are
// terminated (by the process ids this launcher created) and alrun exits
// non-zero.  It stands in for mpirun / jsrun / srun of the reference's test
// and benchmark drivers (test/run_tests.py:109-143).
#include <netinet/in.h>
#include <signal.h>
#include <sys/socket.h>
#include <sys/wait.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

// A listening TCP socket on a free port of the loopback interface.  The launcher keeps it open and
// hands it to rank 0 (AL_MASTER_FD), so no other process can take the port in between.
static int open_rendezvous(int backlog, int* port) {
  int fd = socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return -1;
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  a.sin_port = 0;
  socklen_t len = sizeof(a);
  if (bind(fd, (sockaddr*)&a, sizeof(a)) != 0 || listen(fd, backlog) != 0 || getsockname(fd, (sockaddr*)&a, &len) != 0) {
    close(fd);
    return -1;
  }
  *port = ntohs(a.sin_port);
  return fd;
}

int main(int argc, char** argv) {
  int n = 1, nodes = 0;
  double timeout = 0;
  int i = 1;
  for (; i < argc; ++i) {
    if (!strcmp(argv[i], "-n") && i + 1 < argc) n = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--timeout") && i + 1 < argc) timeout = atof(argv[++i]);
    else if (!strcmp(argv[i], "--nodes") && i + 1 < argc) nodes = atoi(argv[++i]);
    else break;
  }
  if (i >= argc || n < 1 || nodes < 0 || nodes > n) {
    fprintf(stderr, "usage: alrun -n N [--timeout SECONDS] [--nodes K] program [args...]\n");
    return 2;
  }
  const int per_node = nodes > 0 ? (n + nodes - 1) / nodes : n;
  int port = 0;
  const int rendezvous_fd = nodes > 0 ? open_rendezvous(n, &port) : -1;
  if (nodes > 0 && rendezvous_fd < 0) { perror("alrun: rendezvous socket"); return 2; }
  const std::string key = "alrun-" + std::to_string(getpid()) + "-" +
                          std::to_string(std::chrono::steady_clock::now().time_since_epoch().count());
  std::vector<pid_t> kids;
  for (int r = 0; r < n; ++r) {
    pid_t pid = fork();
    if (pid < 0) { perror("fork"); return 2; }
    if (pid == 0) {
      setenv("AL_RANK", std::to_string(r).c_str(), 1);
      setenv("AL_WORLD_SIZE", std::to_string(n).c_str(), 1);
      setenv("AL_LOCAL_RANK", std::to_string(r % per_node).c_str(), 1);
      setenv("AL_JOB_KEY", key.c_str(), 1);
      if (nodes > 0) {
        setenv("AL_TRANSPORT", "tcp", 1);
        setenv("AL_NODE_ID", ("node" + std::to_string(r / per_node)).c_str(), 1);
        setenv("MASTER_ADDR", "127.0.0.1", 1);
        setenv("AL_MASTER_PORT", std::to_string(port).c_str(), 1);
        if (r == 0) setenv("AL_MASTER_FD", std::to_string(rendezvous_fd).c_str(), 1);  // inherited, already listening
        else close(rendezvous_fd);
        // Progress threads are pinned by node-local rank; the modelled nodes share this machine's
        // cores, so equal local ranks would land on one core.  Leave the threads unpinned.
        setenv("AL_PE_BIND", "0", 0);
      }
      execvp(argv[i], argv + i);
      perror("execvp");
      _exit(127);
    }
    kids.push_back(pid);
  }
  if (rendezvous_fd >= 0) close(rendezvous_fd);  // rank 0 holds its own copy
  const auto t0 = std::chrono::steady_clock::now();
  int failures = 0;
  size_t left = kids.size();
  std::vector<bool> done(kids.size(), false);
  while (left) {
    bool progressed = false;
    for (size_t k = 0; k < kids.size(); ++k) {
      if (done[k]) continue;
      int st = 0;
      pid_t w = waitpid(kids[k], &st, WNOHANG);
      if (w == kids[k]) {
        done[k] = true;
        --left;
        progressed = true;
        const bool ok = WIFEXITED(st) && WEXITSTATUS(st) == 0;
        if (!ok) {
          ++failures;
          fprintf(stderr, "alrun: rank %zu %s %d\n", k, WIFSIGNALED(st) ? "killed by signal" : "exited with",
                  WIFSIGNALED(st) ? WTERMSIG(st) : WEXITSTATUS(st));
        }
      }
    }
    const double el = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if ((failures && left) || (timeout > 0 && el > timeout && left)) {
      if (!failures) fprintf(stderr, "alrun: time limit of %.0f s exceeded\n", timeout);
      // give the others a moment to notice and exit on their own, then end them
      std::this_thread::sleep_for(std::chrono::milliseconds(failures ? 2000 : 0));
      for (size_t k = 0; k < kids.size(); ++k)
        if (!done[k] && waitpid(kids[k], nullptr, WNOHANG) == 0) kill(kids[k], SIGKILL);
      for (size_t k = 0; k < kids.size(); ++k)
        if (!done[k]) { waitpid(kids[k], nullptr, 0); done[k] = true; }
      left = 0;
      if (!failures) failures = 1;
    }
    if (!progressed) std::this_thread::sleep_for(std::chrono::milliseconds(5));
  }
  return failures ? 1 : 0;
}
