// ncclras: command-line client of the RAS thread. Connects to the RAS client socket of any
// process of the job (default localhost:28028), asks for a status report and prints it.
//   ncclras [-h host] [-p port] [-t seconds] [-f text|json] [-v] [-m[groups]]   (long forms: --host --port --timeout
//   --format --verbose --monitor[=groups] --help --version); monitor mode prints events until interrupted.
// Reference parity: src/ras/client.cc (options, handshake "CLIENT PROTOCOL", TIMEOUT, STATUS).
#include <getopt.h>
#include <netdb.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <unistd.h>

#include <string>

static bool sendLine(int fd, const std::string& s) {
  std::string l = s + "\n";
  return send(fd, l.data(), l.size(), MSG_NOSIGNAL) == (ssize_t)l.size();
}
static bool readLine(int fd, std::string* out) {
  out->clear();
  char c;
  while (recv(fd, &c, 1, 0) == 1) {
    if (c == '\n') return true;
    out->push_back(c);
  }
  return !out->empty();
}

int main(int argc, char** argv) {
  const char* host = "localhost";
  const char* port = "28028";
  const char* format = "text";
  int timeout = 5;
  bool verbose = false;
  bool monitor = false;
  std::string groups = "all";
  static const struct option longOpts[] = {{"host", required_argument, nullptr, 'h'}, {"port", required_argument, nullptr, 'p'},
                                           {"timeout", required_argument, nullptr, 't'}, {"format", required_argument, nullptr, 'f'},
                                           {"verbose", no_argument, nullptr, 'v'}, {"monitor", optional_argument, nullptr, 'm'},
                                           {"help", no_argument, nullptr, 1}, {"version", no_argument, nullptr, 2}, {nullptr, 0, nullptr, 0}};
  static const char usage[] =
      "usage: %s [OPTION...]\n"
      "  -f, --format=FMT        output format: text (default) or json\n"
      "  -h, --host=HOST         host of the job's RAS client socket (default localhost)\n"
      "  -m, --monitor[=GROUPS]  keep the connection and print events: lifecycle, peers or all (default)\n"
      "  -p, --port=PORT         port of the RAS client socket (default 28028)\n"
      "  -t, --timeout=SECS      how long the serving process waits for the others (default 5)\n"
      "  -v, --verbose           more detail in the report\n"
      "      --help, --version\n";
  int opt;
  while ((opt = getopt_long(argc, argv, "h:p:t:f:vm::", longOpts, nullptr)) != -1) {
    switch (opt) {
      case 'h': host = optarg; break;
      case 'p': port = optarg; break;
      case 't': timeout = atoi(optarg); break;
      case 'f': format = optarg; break;
      case 'v': verbose = true; break;
      case 'm': monitor = true; if (optarg) groups = optarg; break;
      case 1: printf(usage, argv[0]); return 0;
      case 2: printf("ncclras 2.30.7 (nccl_b200)\n"); return 0;
      default:
        fprintf(stderr, usage, argv[0]);
        return 2;
    }
  }
  struct addrinfo hints, *res = nullptr;
  memset(&hints, 0, sizeof(hints));
  hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(host, port, &hints, &res) != 0 || !res) { fprintf(stderr, "ncclras: cannot resolve %s:%s\n", host, port); return 1; }
  int fd = -1;
  for (struct addrinfo* a = res; a; a = a->ai_next) {
    fd = socket(a->ai_family, a->ai_socktype, a->ai_protocol);
    if (fd < 0) continue;
    if (connect(fd, a->ai_addr, a->ai_addrlen) == 0) break;
    close(fd);
    fd = -1;
  }
  freeaddrinfo(res);
  if (fd < 0) { fprintf(stderr, "ncclras: no RAS thread answers at %s:%s (is a job running with NCCL_RAS_ENABLE=1?)\n", host, port); return 1; }
  std::string line;
  if (!sendLine(fd, "CLIENT PROTOCOL 2") || !readLine(fd, &line) || line.compare(0, 15, "SERVER PROTOCOL") != 0) { fprintf(stderr, "ncclras: handshake failed\n"); return 1; }
  if (!sendLine(fd, "TIMEOUT " + std::to_string(timeout)) || !readLine(fd, &line) || line != "OK") { fprintf(stderr, "ncclras: TIMEOUT refused\n"); return 1; }
  if (!sendLine(fd, std::string("SET FORMAT ") + format) || !readLine(fd, &line) || line != "OK") { fprintf(stderr, "ncclras: format %s refused\n", format); return 1; }
  if (monitor) {
    if (!sendLine(fd, "MONITOR " + groups) || !readLine(fd, &line) || line != "OK") { fprintf(stderr, "ncclras: monitor mode refused\n"); return 1; }
    setvbuf(stdout, nullptr, _IOLBF, 0);
  } else if (!sendLine(fd, verbose ? "VERBOSE STATUS" : "STATUS")) return 1;
  char buf[4096];
  ssize_t n;
  while ((n = recv(fd, buf, sizeof(buf), 0)) > 0) fwrite(buf, 1, (size_t)n, stdout);
  close(fd);
  return 0;
}
