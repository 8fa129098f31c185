// Descriptor passing between processes (symm/fd_channel.h): what carries the cuMem VMM chunks of the symmetric memory.
#include <errno.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

#include "symm/fd_channel.h"
#include "tests/host_test.h"

using namespace coccl;

TEST(fd_channel_passes_descriptors_within_and_across_processes) {
  const int fd = memfd_create("coccl-test", MFD_CLOEXEC);
  EXPECT(fd >= 0);
  const char text[] = "chunk zero";
  EXPECT(write(fd, text, sizeof(text)) == (ssize_t)sizeof(text));
  EXPECT_EQ(fdChannelPublish(0x1234, fd), 0);
  // the channel keeps its own duplicate
  close(fd);
  // same process (ranks as threads of one process fetch from their own pid)
  const int mine = fdChannelFetch((int)getpid(), 0x1234, 2000);
  EXPECT(mine >= 0);
  char back[32] = {};
  EXPECT(pread(mine, back, sizeof(text), 0) == (ssize_t)sizeof(text) && strcmp(back, text) == 0);
  close(mine);
  // an unknown key is refused with ENOENT, a process without a channel with a connect error
  EXPECT_EQ(fdChannelFetch((int)getpid(), 0x9999, 2000), -ENOENT);
  EXPECT(fdChannelFetch(1, 0x1234, 500) < 0);
  // another process: the child fetches from the parent's pid, reads the text and appends to the same file
  const pid_t parent = getpid();
  const pid_t child = fork();
  if (child == 0) {
    const int got = fdChannelFetch((int)parent, 0x1234, 5000);
    char buf[32] = {};
    int rc = 1;
    if (got >= 0 && pread(got, buf, sizeof(text), 0) == (ssize_t)sizeof(text) && strcmp(buf, text) == 0 &&
        pwrite(got, "!", 1, sizeof(text)) == 1)
      rc = 0;
    _exit(rc);
  }
  int status = -1;
  EXPECT(waitpid(child, &status, 0) == child && WIFEXITED(status) && WEXITSTATUS(status) == 0);
  const int again = fdChannelFetch((int)getpid(), 0x1234, 2000);
  char mark = 0;
  EXPECT(again >= 0 && pread(again, &mark, 1, sizeof(text)) == 1 && mark == '!');   // one file behind all duplicates
  close(again);
  // withdrawn keys are gone; a second publication under the same key replaces the first
  fdChannelWithdraw(0x1234);
  EXPECT_EQ(fdChannelFetch((int)getpid(), 0x1234, 2000), -ENOENT);
  fdChannelShutdown();
  EXPECT(fdChannelFetch((int)getpid(), 0x1234, 500) < 0);
  // the channel restarts on the next publication
  const int fd2 = memfd_create("coccl-test2", MFD_CLOEXEC);
  EXPECT_EQ(fdChannelPublish(7, fd2), 0);
  close(fd2);
  const int f = fdChannelFetch((int)getpid(), 7, 2000);
  EXPECT(f >= 0);
  close(f);
  fdChannelShutdown();
}
